"""Op layer: dual-number ops (``dual``), torch formulas (``reference``) and
the sm_100a kernel library (``cuda``, ``kernels``, ``build``)."""
