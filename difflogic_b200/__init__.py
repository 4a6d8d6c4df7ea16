"""difflogic_b200 -- the logic-layer hot path of differentiable logic gate networks on NVIDIA B200.

Same Python API as Felix-Petersen/difflogic (`LogicLayer`, `GroupSum`, `PackBitsTensor`,
`CompiledLogicNet`, `functional`), with the CUDA implementation replaced by hand-written
sm_100a kernels behind a C ABI (include/difflogic_b200.h).
"""
from .difflogic import LogicLayer, GroupSum
from .packbitstensor import PackBitsTensor
from .compiled_model import CompiledLogicNet
from . import functional

__all__ = ["LogicLayer", "GroupSum", "PackBitsTensor", "CompiledLogicNet", "functional"]
