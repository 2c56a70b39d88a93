"""ctypes/numpy front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY: imported by tests/, by
__graft_entry__.smoke() and by the cpu_baseline / reference arm of bench.py, never by the
product package.

`Oracle()` wraps liboracle.so (the restatement in oracle.cpp); `Reference()` wraps
oracle/_ref/libref_kernel_test.so (the reference's own kernel_test.cpp functions).
All arrays are float32 C-contiguous numpy arrays in the reference layouts:
softmax MHA tensors (B*S, H*Dh); linear attention Q,K (B*S, D) and V,O (B*S, E).
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_f = C.POINTER(C.c_float)
_z = C.c_size_t


def _p(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f)


def _c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    def __init__(self):
        self.lib = C.CDLL(_build.build_oracle())
        L = self.lib
        L.oracle_num_threads.restype = C.c_int
        L.oracle_set_threads.argtypes = [C.c_int]
        L.oracle_frand.argtypes = [_f, _z, _z]
        L.oracle_mha_fwd.argtypes = [_f, _f, _f, _f, _f, _z, _z, _z, _z, C.c_int]
        L.oracle_mha_bwd.argtypes = [_f] * 8 + [_z] * 4 + [C.c_int]
        L.oracle_linattn_fwd.argtypes = [_f] * 6 + [_z] * 4 + [C.c_int, C.c_int]
        L.oracle_linattn_step1.argtypes = [_f] * 5 + [_z, _z, C.c_int]
        L.oracle_linattn_bwd.argtypes = [_f] * 8 + [_z] * 4 + [C.c_int, C.c_int]
        L.oracle_kernel_attn_bwd.argtypes = [_f] * 9 + [_z] * 4 + [C.c_int]
        L.oracle_phi_elu_fwd.argtypes = [_f, _f, _z, _z, _z]
        L.oracle_phi_elu_bwd.argtypes = [_f, _f, _f, _z, _z, _z]
        L.oracle_rope.argtypes = [_f, _z, _z, _z, _z, C.c_float]
        L.oracle_gelu_exact.argtypes = [_f, _f, _z, C.c_int]

    def num_threads(self):
        return self.lib.oracle_num_threads()

    def set_threads(self, n):
        self.lib.oracle_set_threads(int(n))

    def frand(self, n, skip=0):
        out = np.empty(n, np.float32)
        self.lib.oracle_frand(_p(out), n, skip)
        return out

    def mha_fwd(self, Q, K, V, B, S, H, Dh, f64=False, want_lse=False):
        Q, K, V = _c(Q), _c(K), _c(V)
        O = np.empty_like(Q)
        lse = np.empty(B * H * S, np.float32) if want_lse else None
        self.lib.oracle_mha_fwd(_p(Q), _p(K), _p(V), _p(O), _p(lse), B, S, H, Dh, int(f64))
        return (O, lse) if want_lse else O

    def mha_bwd(self, Q, K, V, O, dO, B, S, H, Dh, f64=False):
        Q, K, V, O, dO = map(_c, (Q, K, V, O, dO))
        dQ, dK, dV = np.empty_like(Q), np.empty_like(Q), np.empty_like(Q)
        self.lib.oracle_mha_bwd(_p(Q), _p(K), _p(V), _p(O), _p(dO), _p(dQ), _p(dK), _p(dV),
                                B, S, H, Dh, int(f64))
        return dQ, dK, dV

    def linattn_fwd(self, Q, K, V, B, S, D, E, elu=True, f64=False):
        """Returns O, den, z_cache.  elu=True: two_stage kernel_attn; elu=False: LinearGPT scan."""
        Q, K, V = _c(Q), _c(K), _c(V)
        O = np.empty((B * S, E), np.float32)
        den = np.empty(B * S, np.float32)
        zc = np.empty((B * S, D), np.float32)
        self.lib.oracle_linattn_fwd(_p(Q), _p(K), _p(V), _p(O), _p(den), _p(zc), B, S, D, E,
                                    int(elu), int(f64))
        return O, den, zc

    def linattn_step1(self, O, dO, den, f64=False):
        O, dO, den = _c(O), _c(dO), _c(den)
        N, E = O.shape
        dnum = np.empty_like(O)
        dden = np.empty(N, np.float32)
        self.lib.oracle_linattn_step1(_p(O), _p(dO), _p(den), _p(dnum), _p(dden), N, E, int(f64))
        return dnum, dden

    def linattn_bwd(self, Q, K, V, dnum, dden, B, S, D, E, elu=True, f64=False):
        Q, K, V, dnum, dden = map(_c, (Q, K, V, dnum, dden))
        dQ = np.empty((B * S, D), np.float32)
        dK = np.empty((B * S, D), np.float32)
        dV = np.empty((B * S, E), np.float32)
        self.lib.oracle_linattn_bwd(_p(Q), _p(K), _p(V), _p(dnum), _p(dden), _p(dQ), _p(dK), _p(dV),
                                    B, S, D, E, int(elu), int(f64))
        return dQ, dK, dV

    def kernel_attn_bwd(self, Q, K, V, O, dO, den, B, S, D, E, f64=False):
        Q, K, V, O, dO, den = map(_c, (Q, K, V, O, dO, den))
        dQ = np.empty((B * S, D), np.float32)
        dK = np.empty((B * S, D), np.float32)
        dV = np.empty((B * S, E), np.float32)
        self.lib.oracle_kernel_attn_bwd(_p(Q), _p(K), _p(V), _p(O), _p(dO), _p(den),
                                        _p(dQ), _p(dK), _p(dV), B, S, D, E, int(f64))
        return dQ, dK, dV

    def phi_elu_fwd(self, x, D):
        x = _c(x)
        N, E = x.shape
        phi = np.empty((N, D), np.float32)
        self.lib.oracle_phi_elu_fwd(_p(x), _p(phi), N, D, E)
        return phi

    def phi_elu_bwd(self, dphi, x):
        dphi, x = _c(dphi), _c(x)
        N, D = dphi.shape
        E = x.shape[1]
        dx = np.empty((N, E), np.float32)
        self.lib.oracle_phi_elu_bwd(_p(dphi), _p(x), _p(dx), N, D, E)
        return dx

    def rope(self, X, S, head_dim, sign=1.0):
        X = _c(X).copy()
        rows, D = X.shape
        self.lib.oracle_rope(_p(X), rows, S, D, head_dim, float(sign))
        return X

    def gelu_exact(self, A, deriv=False):
        A = _c(A)
        out = np.empty_like(A)
        self.lib.oracle_gelu_exact(_p(A), _p(out), A.size, int(deriv))
        return out


class Reference:
    """The reference's own CPU functions (kernel_test.cpp), compiled from the reference tree."""

    def __init__(self):
        path = _build.build_reference()
        if path is None:
            raise FileNotFoundError("oracle/_ref/libref_kernel_test.so is not built and the "
                                    "reference tree is not mounted")
        self.lib = C.CDLL(path)
        L = self.lib
        L.ref_frand.argtypes = [_f, _z, _z]
        L.ref_mha_fwd_all.argtypes = [_f] * 4 + [_z] * 4
        L.ref_mha_bwd_all.argtypes = [_f] * 8 + [_z] * 4
        L.ref_kernel_attn_fwd_all.argtypes = [_f] * 5 + [_z] * 4
        L.ref_kernel_attn_bwd_all.argtypes = [_f] * 9 + [_z] * 4

    @staticmethod
    def available():
        return _build.build_reference() is not None

    def frand(self, n, skip=0):
        out = np.empty(n, np.float32)
        self.lib.ref_frand(_p(out), n, skip)
        return out

    def mha_fwd(self, Q, K, V, B, S, H, Dh):
        Q, K, V = _c(Q), _c(K), _c(V)
        O = np.empty_like(Q)
        self.lib.ref_mha_fwd_all(_p(Q), _p(K), _p(V), _p(O), B, S, H, Dh)
        return O

    def mha_bwd(self, Q, K, V, O, dO, B, S, H, Dh):
        Q, K, V, O, dO = map(_c, (Q, K, V, O, dO))
        dQ, dK, dV = np.empty_like(Q), np.empty_like(Q), np.empty_like(Q)
        self.lib.ref_mha_bwd_all(_p(Q), _p(K), _p(V), _p(O), _p(dO), _p(dQ), _p(dK), _p(dV),
                                 B, S, H, Dh)
        return dQ, dK, dV

    def kernel_attn_fwd(self, Q, K, V, B, S, D, E):
        Q, K, V = _c(Q), _c(K), _c(V)
        O = np.empty((B * S, E), np.float32)
        den = np.empty(B * S, np.float32)
        self.lib.ref_kernel_attn_fwd_all(_p(Q), _p(K), _p(V), _p(O), _p(den), B, S, D, E)
        return O, den

    def kernel_attn_bwd(self, Q, K, V, O, dO, den, B, S, D, E):
        Q, K, V, O, dO, den = map(_c, (Q, K, V, O, dO, den))
        dQ = np.empty((B * S, D), np.float32)
        dK = np.empty((B * S, D), np.float32)
        dV = np.empty((B * S, E), np.float32)
        self.lib.ref_kernel_attn_bwd_all(_p(Q), _p(K), _p(V), _p(O), _p(dO), _p(den),
                                         _p(dQ), _p(dK), _p(dV), B, S, D, E)
        return dQ, dK, dV


class ReferenceCuda:
    """The reference's own CUDA kernels (two_stage_cuda_kernels.cu, linear_cuda_kernels.cu compiled
    unmodified for sm_100, see ref_cuda_wrap.cu), on torch CUDA float tensors.  Used by the GPU
    tests as a second checker and by the benchmark to time the reference's serial-scan kernels."""

    def __init__(self):
        path = _build.build_reference_cuda()
        if path is None:
            raise FileNotFoundError("oracle/_ref/libref_cuda.so is not built and the reference tree is not mounted")
        self.lib = C.CDLL(path)
        vp = C.c_void_p
        self.lib.refcuda_mha_fwd.argtypes = [vp] * 4 + [_z] * 4
        self.lib.refcuda_mha_bwd.argtypes = [vp] * 8 + [_z] * 4
        self.lib.refcuda_kernel_attn_fwd_bwd.argtypes = [vp] * 14 + [_z] * 4 + [C.c_int]
        self.lib.refcuda_linear_fwd_bwd.argtypes = [vp] * 14 + [_z] * 4 + [C.c_int]

    @staticmethod
    def available():
        return _build.build_reference_cuda() is not None

    def mha_fwd(self, Q, K, V, O, B, S, H, Dh):
        assert self.lib.refcuda_mha_fwd(*(t.data_ptr() for t in (Q, K, V, O)), B, S, H, Dh) == 0

    def mha_bwd(self, Q, K, V, O, dO, dQ, dK, dV, B, S, H, Dh):
        assert self.lib.refcuda_mha_bwd(*(t.data_ptr() for t in (Q, K, V, O, dO, dQ, dK, dV)), B, S, H, Dh) == 0

    def scan_buffers(self, B, S, D, E, device):
        """Outputs and scratch of one forward + backward of either linear flavour."""
        import torch
        N = B * S
        f = lambda *s: torch.empty(*s, device=device, dtype=torch.float32)
        return dict(O=f(N, E), den=f(N), dQ=f(N, D), dK=f(N, D), dV=f(N, E), zc=f(N, D), Sbuf=f(B * max(D, E), max(D, E)),
                    zbuf=f(B, D), dnum=f(N, E), dden=f(N))

    def _scan(self, fn, Q, K, V, dO, buf, B, S, D, E, bwd):
        order = ("O", "den", "dQ", "dK", "dV", "zc", "Sbuf", "zbuf", "dnum", "dden")
        ptrs = [t.data_ptr() for t in (Q, K, V, dO)] + [buf[k].data_ptr() for k in order]
        assert fn(*ptrs, B, S, D, E, int(bwd)) == 0

    def kernel_attn(self, Q, K, V, dO, buf, B, S, D, E, bwd=True):
        self._scan(self.lib.refcuda_kernel_attn_fwd_bwd, Q, K, V, dO, buf, B, S, D, E, bwd)

    def linear(self, Qp, Kp, V, dO, buf, B, S, D, E, bwd=True):
        self._scan(self.lib.refcuda_linear_fwd_bwd, Qp, Kp, V, dO, buf, B, S, D, E, bwd)
