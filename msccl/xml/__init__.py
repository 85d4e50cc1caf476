"""MSCCL-IR XML: typed loader and static validator."""
from msccl.xml.loader import AlgoIR, GpuIR, StepIR, TbIR, load_xml, load_xml_file, load_plan_table  # noqa: F401
from msccl.xml.validator import validate  # noqa: F401
