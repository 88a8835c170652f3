"""Matrix products of the parts: picks the kernel for a contraction out[m, n] = sum_k a[m, k] w[n, k].

bfloat16 activations and weights whose shapes the tensor-core kernel accepts go to the tcgen05
kernel; everything else -- the whole float32 path, mixed dtypes, odd shapes -- goes to the FP32-pipe
kernel, which accepts any size.  Either way accumulation is float32.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K

MODE_STORE, MODE_ADD, MODE_SWIGLU = K.MODE_STORE, K.MODE_ADD, K.MODE_SWIGLU

# set to False to force the FP32-pipe kernel everywhere (tests compare the two)
use_tensor_cores = True
# set to False to keep dense products with many tokens on the single-CTA kernel
use_paired_kernel = True


def project(a, w, out, mode=MODE_STORE, **kw):
    """Dense or grouped projection; see csrc/lib.py: gemm_simt for the keyword arguments."""
    if use_tensor_cores and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        # products with many tokens go to the two-SM kernel, dense or grouped (it refuses, launching nothing,
        # what it does not take: few tokens per group, features that are no multiple of 256, a row gather)
        if use_paired_kernel and "a_rows" not in kw and kw.get("m_rows", a.shape[0]) >= 512 \
                and K.gemm_tc_pair(a, w, out, mode, **kw):
            return
        if K.gemm_tc(a, w, out, mode, **kw):
            return
    K.gemm_simt(a, w, out, mode, **kw)
