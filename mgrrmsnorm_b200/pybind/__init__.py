"""Home of the compiled torch extension `rmsnorm_cuda_ops` (source: pytorch_binding/binding.cpp).

`python setup.py build_ext --inplace` (or `python -m mgrrmsnorm_b200.build --binding`) places
`rmsnorm_cuda_ops.*.so` here. It is the same binding the reference ships as its top-level module
`rmsnorm_cuda_ops` (pytorch_binding/binding.cpp:136-139), linked against lib/libmgr_b200.so.
`mgrrmsnorm_b200.rmsnorm_cuda_ops` uses it when it is present and the ctypes route otherwise.
"""
