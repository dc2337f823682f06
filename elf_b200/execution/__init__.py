"""Runtime: blocks, schedule interpreter, remat, activation offload, p2p channels."""

from .block import PipelineBlock, Variable
from .engine import Engine, compute_loss
from .remat import RematManager
from .offload import OffloadToCPU, PinnedHostTensorPool, OffloadManager
from .channels import Channel, ChannelTable

__all__ = ["PipelineBlock", "Variable", "Engine", "compute_loss", "RematManager", "OffloadToCPU", "PinnedHostTensorPool", "OffloadManager", "Channel", "ChannelTable"]
