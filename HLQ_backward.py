"""``import HLQ_backward`` from the repository root resolves to the B200 implementation, so the
reference's latency harness (cuda_measure/measure.py:16,65,72) runs against it unchanged."""
from hot_b200.HLQ_backward import backward  # noqa: F401
