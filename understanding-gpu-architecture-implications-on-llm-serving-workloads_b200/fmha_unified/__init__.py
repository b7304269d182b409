import torch
from . import _C, ops
