"""Stand-ins for the reference's three native modules, with the signatures of its pybind11 bindings
(reference: gact/setup.py:4-22 builds ``gact.cpp_extension.minimax``, ``.quantization`` and ``.calc_precision``).

Python written against those modules - the reference's own ``ops.py`` and ``autoprec.py`` import them as
``ext_minimax``, ``ext_quantization`` and ``ext_calc_precision`` - runs on ``libgact_b200.so`` through these shims.
They always use the reference's random stream (``curand`` mode), so the packed bytes equal the reference's for the
same seed.  The package's own hot path (``gact.ops``) does not go through here: it calls the fused entry points
directly and skips the padding copy and the separate min/max pass.
"""
