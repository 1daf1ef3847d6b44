"""B200 (sm_100a) implementation of the structured-matmul operators of pabillam/mem-efficient-blr.

The operator modules keep the reference's function names and argument layouts
(``blast_kernels``, ``blast_sym_quant_kernels``, ``monarch_kernels``, ``low_rank_kernels``,
``dense_kernels``), so a YAML ``func:`` path only changes its module prefix.  All arithmetic runs in
hand-written CUDA behind the C ABI declared in ``include/blr_b200.h``; there is no CPU or Triton
fallback: importing an operator without the built library raises.
"""
__version__ = "0.1.0"
