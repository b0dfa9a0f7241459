from .accuracy import SQNR_THRESHOLD_DB, bf16_ulp_mismatch, bitwise_equal, check_determinism, check_input_readonly, sqnr_db
from .bench import bench_kernel
from .roofline import RooflineResult, measure_roofline

__all__ = [
    "RooflineResult",
    "SQNR_THRESHOLD_DB",
    "bench_kernel",
    "bf16_ulp_mismatch",
    "bitwise_equal",
    "check_determinism",
    "check_input_readonly",
    "measure_roofline",
    "sqnr_db",
]
