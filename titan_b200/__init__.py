"""titan_b200: a Blackwell (sm_100a) native LLM training framework.

PyTorch is the framework layer; the hot operators are hand-written CUDA kernels for B200
(tcgen05 tensor cores with TMEM accumulators, TMA tile movement, peer-memory collectives over
NVLink 5 / NVSwitch), opted into per recipe through model converters.
"""

__version__ = "0.1.0"
