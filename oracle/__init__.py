"""CPU oracle for the structured-matmul path (test infrastructure only).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this
package.  The product package never does; it fails loudly without its CUDA library.
"""
