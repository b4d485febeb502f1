"""cverl_b200: a Blackwell-native (sm_100a) RL post-training framework.

PyTorch is the framework layer; the hot operators are hand-written CUDA
kernels (tcgen05 / TMEM / TMA) loaded from ``cverl_b200/lib`` and the host
runtime (public C ABI, topology, IO, tokenizers, transports) is C++.
"""
__version__ = "0.1.0"
