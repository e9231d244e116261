from .clocks import ClockSampler  # noqa: F401
from .timing import l2_flush, time_cuda  # noqa: F401
