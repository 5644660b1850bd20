"""Op implementations: ``_impl/<op>/`` belongs to the op module ``cake.<op>``.

An op's package calls ``loader.install_op("<op>")`` at import and defines its entry points (the op's ``OP.exports``),
``prebuild(*, device=None, max_workers=None, **model_params)`` and ``release()``.  It reads its variant and options
when a call runs (``config.variant`` / ``config.option``), takes scratch from ``workspace.take`` and never reads the
environment (reference: miles_ext_kernels/cake/_impl/__init__.py:1-7).
"""
