"""CPU oracle for the LANS optimizer op.  TEST INFRASTRUCTURE ONLY.

NumPy restatement of the reference's multi-tensor LANS step.  Only the tests,
the smoke check and the benchmark's CPU baseline leg may import it.

Follows src/op/dialect/cuda/kernels/multi_tensor_lans.cu:207-322 (stage 1),
:326-399 (stage 2), :401-450 (pass order) and the host-side bias correction of
src/op/dialect/cuda/lans.cc:108-117.  The reference's per-tensor scratch slices
overlap for three or more tensors (lans.cc:126-129 uses numels[i-1] instead of
a prefix sum); this oracle implements the intended, non-overlapping semantics
(NVIDIA apex FusedLANS, which tests/python/optim/test_lans.py:18-21 compares
with).  apex is not available here.  Parity pin: tests/test_ref_kernels_gpu.py
runs the reference's own multi_tensor_lans.cu (compiled unmodified by
oracle/ref_build/build_ref.py) on the GPU and holds this oracle and the product's
kernels to rel 1e-5 against it over consecutive steps and all flag combinations.
"""
import numpy as np


def bias_corrections(step, beta1, beta2, bias_correction=1):
    """lans.cc:108-113: 1 - std::pow(float beta, int step), evaluated in double
    (the C++ overload promotes) and stored as float; 1.0 when disabled."""
    if bias_correction == 1:
        return (np.float32(1.0 - float(np.float32(beta1)) ** int(step)),
                np.float32(1.0 - float(np.float32(beta2)) ** int(step)))
    return np.float32(1.0), np.float32(1.0)


def lans_step(g, p, m, v, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-6,
              bias_correction=1, weight_decay=0.01, grad_averaging=1, mode=1,
              normalize_grad=True, dtype=np.float32):
    """One LANS step over lists of arrays; returns new (p, m, v) lists.

    `dtype` float32 reproduces the kernel arithmetic order; float64 gives the
    high-precision cross-check.
    """
    T = dtype
    bc1, bc2 = bias_corrections(step, beta1, beta2, bias_correction)
    bc1, bc2 = T(bc1), T(bc2)
    b1, b2, e_, wd, lr_ = T(np.float32(beta1)), T(np.float32(beta2)), T(np.float32(eps)), \
        T(np.float32(weight_decay)), T(np.float32(lr))
    b3 = T(1) - b1 if grad_averaging == 1 else T(1)           # lans.cc:114-117
    new_p, new_m, new_v = [], [], []
    for gi, pi, mi, vi in zip(g, p, m, v):
        gi = gi.astype(T); pi = pi.astype(T); mi = mi.astype(T); vi = vi.astype(T)
        gnorm = T(np.sqrt(np.sum(gi.astype(np.float64) ** 2)))
        pnorm = T(np.sqrt(np.sum(pi.astype(np.float64) ** 2)))
        sg = gi
        if normalize_grad and gnorm != 0:
            sg = gi / (gnorm + e_)                            # multi_tensor_lans.cu:283-286
        if mode == 0:                                         # :287-297 (L2 on scaled grad)
            sg = sg + wd * pi
            mi = mi * b1 + b3 * sg
            vi = vi * b2 + (T(1) - b2) * sg * sg
            denom = np.sqrt(vi / bc2) + e_
            um = (mi / bc1) / denom
            ug = sg / denom
        else:                                                 # :298-307 (decoupled decay)
            mi = mi * b1 + b3 * sg
            vi = vi * b2 + (T(1) - b2) * sg * sg
            denom = np.sqrt(vi / bc2) + e_
            sp = wd * pi
            um = (mi / bc1) / denom + sp
            ug = sg / denom + sp
        umn = T(np.sqrt(np.sum(um.astype(np.float64) ** 2)))
        ugn = T(np.sqrt(np.sum(ug.astype(np.float64) ** 2)))
        rm = lr_ * (pnorm / umn) if (umn != 0 and pnorm != 0) else lr_   # :346-349
        rg = lr_ * (pnorm / ugn) if (ugn != 0 and pnorm != 0) else lr_
        rm = rm * b1
        rg = rg * b3
        pi = pi - rm * um - rg * ug                           # :383
        new_p.append(pi.astype(T)); new_m.append(mi.astype(T)); new_v.append(vi.astype(T))
    return new_p, new_m, new_v
