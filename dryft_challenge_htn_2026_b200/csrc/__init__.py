"""CUDA sources for sm_100a (``*.cu``), their build step (``build``) and ctypes entry points (``api``)."""
