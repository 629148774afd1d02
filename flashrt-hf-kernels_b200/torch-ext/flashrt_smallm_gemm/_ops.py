import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from flashrt_b200_core import make_ops  # noqa: E402

ops, add_op_namespace_prefix = make_ops("flashrt_smallm_gemm_b200")
