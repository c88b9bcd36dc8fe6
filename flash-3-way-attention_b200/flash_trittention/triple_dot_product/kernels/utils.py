"""Window-argument helper shared by the entry point and the dense PyTorch module.

Mirrors ``process_masking_variables`` of the reference
(``src/flash_trittention/triple_dot_product/kernels/utils.py:6-17``): a window given as
``None`` spans the whole sequence.
"""
from typing import Optional


def process_masking_variables(
    seq_len: int,
    k1_window: Optional[int] = None,
    k2_window: Optional[int] = None,
    kk_left: Optional[int] = None,
    kk_right: Optional[int] = None,
):
    pick = lambda w: seq_len if w is None else w
    return pick(k1_window), pick(k2_window), pick(kk_left), pick(kk_right)
