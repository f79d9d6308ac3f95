"""Host-side mirror of HGCalML's ``modules/index_replacer_op.py``."""
from __future__ import annotations

import torch

from . import _capi as C


def IndexReplacer(to_be_replaced, replacements):
    """``out[i] = replacements[to_be_replaced[i]]``, negative entries pass through
    (modules/index_replacer_op.py:6-15).  Entries beyond the table keep the value 0 the output is
    created with (the reference leaves them unwritten)."""
    C.require_cuda(to_be_replaced, replacements)
    tbr, rep = C.i32(to_be_replaced), C.i32(replacements)
    out = torch.zeros_like(tbr)
    C.check(C.lib.hgc_index_replacer(C.ptr(tbr), C.ptr(rep), C.ptr(out), tbr.numel(), rep.shape[0],
                                     None, C.stream_of(tbr)), "IndexReplacer")
    return out
