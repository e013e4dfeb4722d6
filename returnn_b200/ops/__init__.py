"""
Hot ops. Each module exposes a functional API on raw ``torch.Tensor`` s with autograd support.
On CUDA tensors the hand-written sm_100a kernels from ``librb200.so`` run; on CPU a torch implementation of the same
math (which is also the numerics oracle in the tests).
"""
