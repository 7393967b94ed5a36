from lasp_b200.utils import *  # noqa: F401,F403
from lasp_b200.utils import build_slope_tensor, get_memory  # noqa: F401
