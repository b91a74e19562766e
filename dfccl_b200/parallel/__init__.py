from .groups import Dist, init_distributed
from .ddp import DaemonDDP
from .graph import GraphedStep
