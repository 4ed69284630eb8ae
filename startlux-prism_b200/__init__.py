"""prism_b200: the quantized linear-layer hot path of StartLux-Prism for the B200 (sm_100a).

Python host code with the reference's operator API (kernels/w8a8.py, quant.py, w4a8.py, mxfp4.py, tp.py,
gguf_weights.py) over a C-ABI CUDA library (csrc/, include/prism_b200.h).  There is no Triton path, no other-GPU path
and no CPU fallback: an operator raises if the library is not built or a kernel cannot take its arguments.
"""
__version__ = "0.1.0"
