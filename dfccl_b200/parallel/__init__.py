from .groups import Dist, init_distributed
from .ddp import DaemonDDP
