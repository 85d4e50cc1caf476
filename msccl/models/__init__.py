"""Model blocks of the benchmark configurations, built from ``msccl.parallel``."""
from msccl.models.blocks import llama3_8b_mlp, moe_block_64x2  # noqa: F401
