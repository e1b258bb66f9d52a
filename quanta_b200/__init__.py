"""quanta_b200 — the quantized-inference path of zelez-lab/quanta, B200-native.

Host-side mirror of the reference API (``quanta::sci::quant`` in ``quant``,
``quanta::nn::quant`` in ``nn_quant``) over the C ABI of ``libqb200.so``
(``include/qb200.h``).  All compute is hand-written CUDA for sm_100a; there is
no CPU path.
"""
from . import _lib
from ._lib import IN_OUT, OUT_IN
from .quant import (Block, Granularity, Group, PerChannel, PerTensor, QuantDtype, QuantError, QuantizedMatrix,
                    granularity_from_grid)
from .nn_quant import (FORMAT_VERSION, LoadedQuant, LoadedSafetensors, QuantLeaf, QuantizedLinear, load, load_named,
                       load_named_f32, quantize_named, save_named)

__all__ = [
    "Block", "Granularity", "Group", "PerChannel", "PerTensor", "QuantDtype", "QuantError", "QuantizedMatrix",
    "granularity_from_grid", "FORMAT_VERSION", "LoadedQuant", "LoadedSafetensors", "QuantLeaf", "QuantizedLinear",
    "load", "load_named", "load_named_f32", "quantize_named", "save_named", "IN_OUT", "OUT_IN",
]
