"""nanoserve_b200: the continuous-batching forward hot path of nanoserve, rebuilt for B200 (sm_100a).

Host logic (scheduler, paged KV manager, engine, CUDA-graph runners) is Python with the reference's class and
method names; every device op the reference wrote in Triton is a hand-written CUDA kernel in
lib/libnanoserve_b200.so, reached through the C ABI of include/nanoserve_b200.h (see _lib.py).
"""
__version__ = "0.1.0"
