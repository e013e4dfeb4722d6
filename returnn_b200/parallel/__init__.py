"""
Data-parallel machinery: flat parameter / gradient arena, bucketed gradient reduction overlapped with backward,
parameter averaging, symmetric (peer-mapped) memory and the fused NVLink collectives.
"""
