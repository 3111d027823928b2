"""InterOp DSL: describe a cross-cluster collective as staged operations,
check it symbolically, and emit the per-rank XML plans that the C2C planner
executes (FLAGCX_C2C_ALGO=XML_INPUT)."""
from .algorithm import *  # noqa: F401,F403
