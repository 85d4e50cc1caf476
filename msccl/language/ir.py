"""Import path kept for programs written against msccl-tools (``msccl.language.ir``); the code lives in ``msccl.language.mscclir``."""
from msccl.language.mscclir import *  # noqa: F401,F403
from msccl.language.xmlwriter import ir_to_xml  # noqa: F401,E402
