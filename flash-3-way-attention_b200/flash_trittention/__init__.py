"""flash_trittention for NVIDIA B200: three-way attention on hand-written sm_100a kernels.

Same public names as the reference package (``src/flash_trittention/__init__.py:11-26``):
``flash_trittention`` (triple-dot-product) and ``TrittentionTriton`` (dot-product-sum),
imported lazily so that ``import flash_trittention`` works without a GPU.
"""

__version__ = "0.1.0"

__all__ = ["flash_trittention", "TrittentionTriton"]  # the reference's public names; TrittentionTDP is an extra

_LAZY_ATTRS = {
    "flash_trittention": (".triple_dot_product.flash_trittention", "flash_trittention"),
    "TrittentionTriton": (".dot_product_sum.trittention_triton", "TrittentionTriton"),
    "TrittentionTDP": (".ops", "TrittentionTDP"),  # torch.library operators + module (not in the reference)
    # raises if a kernel of an earlier call gave up on a bounded barrier wait (not in the reference)
    "check_status": ("._native", "check_status"),
}


def __getattr__(name):
    try:
        module_path, attr = _LAZY_ATTRS[name]
    except KeyError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
    from importlib import import_module

    value = getattr(import_module(module_path, __name__), attr)
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_LAZY_ATTRS))
