"""B200-native sparse Mixture-of-Experts decode reader.

Host-side Python mirrors the reference operator API
(`calibration_free_moe.reader.{budget,sketch,progressive}`); all decode-time
arithmetic runs in the hand-written sm_100a CUDA library under `csrc/`, reached
through its C ABI (`include/cfm_b200.h`).
"""

__version__ = "0.1.0"
