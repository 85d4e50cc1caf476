"""MSCCLang: chunk-oriented DSL for collective algorithms, compiled to MSCCL-IR XML.

``from msccl.language import *`` provides the same names as the reference package
(reference ``msccl/language/__init__.py``): ``MSCCLProgram``, ``chunk``, ``XML``, ``Check``,
``Ref``, ``Buffer``, ``Instruction``, ``ThreadblockPolicy``, ``ir_to_xml`` ...
"""
from collections import defaultdict  # noqa: F401  (programs written for the reference rely on it)

from msccl.language.mscclir import (Buffer, ChunkInstruction, ChunkRef, Gpu, Instruction, Op, Program,
                                    Threadblock, ThreadblockPolicy)
from msccl.language.symbolic import BufferSlice, Chunk, ReduceChunk
from msccl.language.dag import InstructionDAG
from msccl.language.compiler.schedule import (auto_assign_tbs, channel_assignment, manual_assign_tbs,
                                              topo_sort_instrs)
from msccl.language.compiler.verify import check_dependency_cycles, check_threadblock_ordering
from msccl.language.xmlwriter import ir_to_xml
from msccl.language.program import (MSCCLProgram, Ref, chunk, create_scratch, XML, Check, Print, _curr)
import msccl.collectives as collectives  # noqa: F401
