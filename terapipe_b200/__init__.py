"""terapipe_b200: token-level pipeline parallel training of causal Transformers on B200.

Sub-packages: ``models`` (configs, layer, slicing), ``parallel`` (groups, tensor-parallel
layers, pipeline links, symmetric memory), ``ops`` (sm_100a CUDA kernels and their
Python bindings), ``runtime`` (portable autograd pipeline and the B200 engine),
``planner`` (latency / FLOP / memory models and the slice-schedule dynamic program),
``utils``.
"""
__version__ = "0.1.0"
