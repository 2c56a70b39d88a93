"""Python front end of libcxxattn.so, used by the tests and the benchmark.

The product is the shared library and its C-ABI (include/cxxattn.h); this module only binds
it with ctypes and mirrors the reference's kernel entry points by name and argument order
(`two_stage_cuda.*` = src/TwoStage/two_stage_cuda_kernels.cuh:18-85, `linear_cuda.*` =
src/LinearAttention/linear_cuda_kernels.cuh:11-46) on torch CUDA tensors, which stand in for
TensorN::CudaTensor<float>.  torch supplies device memory and streams, nothing else: there is no
fallback, and loading fails loudly when the library has not been built.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# CXXATTN_LIBRARY points the binding at another build of the same C-ABI (an experimental variant).
LIB_PATH = os.environ.get("CXXATTN_LIBRARY") or os.path.join(_HERE, "libcxxattn.so")

F32, BF16 = 0, 1
MAP_NONE, MAP_ELU1 = 0, 1

SYMBOLS = [
    "cxxattn_strerror", "cxxattn_version",
    "cxxattn_mha_fwd", "cxxattn_mha_bwd_workspace_bytes", "cxxattn_mha_bwd",
    "cxxattn_linattn_workspace_bytes", "cxxattn_linattn_fwd", "cxxattn_linattn_bwd_step1",
    "cxxattn_linattn_bwd_dq", "cxxattn_linattn_bwd_dkdv", "cxxattn_linattn_bwd",
    "cxxattn_phi_elu_fwd", "cxxattn_phi_elu_bwd", "cxxattn_rope", "cxxattn_gelu_exact",
    "cxxattn_sync_status", "cxxattn_last_timeout_site", "cxxattn_cast", "cxxattn_rope_cast", "cxxattn_rope_cast_pair",
    "cxxattn_linattn_decode_step", "cxxattn_mha_decode_workspace_bytes", "cxxattn_mha_decode_step",
    "cxxattn_selftest_umma",
    "cxxattn_host_plan_create", "cxxattn_host_plan_destroy", "cxxattn_mha_fwd_bwd_host",
    "cxxattn_linattn_fwd_noalloc", "cxxattn_linattn_noalloc_capacity", "cxxattn_set_timing_events",
    "cxxattn_lin_host_plan_create", "cxxattn_lin_host_plan_destroy", "cxxattn_linattn_fwd_bwd_host",
    "cxxattn_set_option", "cxxattn_get_option", "cxxattn_selftest_wait_limit", "cxxattn_adamw_step",
    "cxxattn_adamw_step_mixed", "cxxattn_adamw_step_exchange",
    "cxxattn_colsum_workspace_bytes", "cxxattn_colsum", "cxxattn_layernorm_bwd_workspace_bytes", "cxxattn_layernorm_bwd", "cxxattn_peer_alloc", "cxxattn_peer_free", "cxxattn_peer_export", "cxxattn_peer_open", "cxxattn_peer_close",
]

# cxxattn_set_option keys (include/cxxattn.h)
OPT_FWD_LATE_WAIT, OPT_BWD_PERSISTENT, OPT_LIN_GROUPS, OPT_LIN_SIDE_STREAM = 0, 1, 2, 3


class MhaDesc(C.Structure):
    _fields_ = [("B", C.c_int64), ("S", C.c_int64), ("H", C.c_int64), ("Dh", C.c_int64),
                ("stride_b", C.c_int64), ("stride_s", C.c_int64), ("stride_h", C.c_int64),
                ("dtype", C.c_int32), ("reserved", C.c_int32)]


class LinDesc(C.Structure):
    _fields_ = [("B", C.c_int64), ("S", C.c_int64), ("D", C.c_int64), ("E", C.c_int64),
                ("dtype", C.c_int32), ("feature_map", C.c_int32), ("eps_in_den", C.c_int32),
                ("ld_qk", C.c_int32)]


class CxxAttnError(RuntimeError):
    def __init__(self, code, what):
        super().__init__(f"{what}: {strerror(code)} ({code})")
        self.code = code


_lib = None


def lib():
    """The loaded C-ABI library.  Raises if it has not been built (python cxx-gpt_b200/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(f"{LIB_PATH} is missing: build it with `python cxx-gpt_b200/build.py`; "
                                    "there is no fallback path")
        L = C.CDLL(LIB_PATH)
        vp, sz, i32, f32p = C.c_void_p, C.c_size_t, C.c_int, C.c_void_p
        L.cxxattn_strerror.restype = C.c_char_p
        L.cxxattn_strerror.argtypes = [i32]
        L.cxxattn_version.restype = C.c_char_p
        L.cxxattn_mha_fwd.argtypes = [C.POINTER(MhaDesc), vp, vp, vp, vp, f32p, vp]
        L.cxxattn_mha_bwd_workspace_bytes.restype = sz
        L.cxxattn_mha_bwd_workspace_bytes.argtypes = [C.POINTER(MhaDesc), i32]
        L.cxxattn_mha_bwd.argtypes = [C.POINTER(MhaDesc)] + [vp] * 9 + [vp, sz, vp]
        L.cxxattn_linattn_workspace_bytes.restype = sz
        L.cxxattn_linattn_workspace_bytes.argtypes = [C.POINTER(LinDesc)]
        L.cxxattn_linattn_fwd.argtypes = [C.POINTER(LinDesc)] + [vp] * 6 + [vp, sz, vp]
        L.cxxattn_linattn_bwd_step1.argtypes = [vp] * 5 + [sz, sz, vp]
        L.cxxattn_linattn_bwd_dq.argtypes = [C.POINTER(LinDesc)] + [vp] * 7 + [vp, sz, vp]
        L.cxxattn_linattn_fwd.restype = L.cxxattn_linattn_bwd_dq.restype = L.cxxattn_linattn_bwd_dkdv.restype = i32
        L.cxxattn_linattn_bwd_dkdv.argtypes = [C.POINTER(LinDesc)] + [vp] * 7 + [vp, sz, vp]
        L.cxxattn_linattn_bwd.argtypes = [C.POINTER(LinDesc)] + [vp] * 9 + [vp, sz, vp]
        L.cxxattn_phi_elu_fwd.argtypes = [vp, vp, sz, sz, sz, vp]
        L.cxxattn_phi_elu_bwd.argtypes = [vp, vp, vp, sz, sz, sz, vp]
        L.cxxattn_rope.argtypes = [vp, vp, sz, sz, sz, sz, C.c_float, vp]
        L.cxxattn_gelu_exact.argtypes = [vp, vp, sz, i32, vp]
        L.cxxattn_cast.argtypes = [vp, i32, vp, i32, sz, vp]
        L.cxxattn_rope_cast.argtypes = [vp, i32, vp, i32, sz, sz, sz, sz, C.c_float, vp]
        L.cxxattn_rope_cast_pair.argtypes = [vp, vp, i32, vp, vp, i32, sz, sz, sz, sz, C.c_float, vp]
        L.cxxattn_linattn_decode_step.argtypes = [C.POINTER(LinDesc)] + [vp] * 7 + [vp]
        L.cxxattn_mha_decode_workspace_bytes.restype = sz
        L.cxxattn_mha_decode_workspace_bytes.argtypes = [C.POINTER(MhaDesc)]
        L.cxxattn_mha_decode_step.argtypes = [C.POINTER(MhaDesc)] + [vp] * 5 + [C.c_int64, vp, vp, sz, vp]
        L.cxxattn_sync_status.argtypes = [vp]
        L.cxxattn_set_timing_events.argtypes = [vp, vp]
        L.cxxattn_set_timing_events.restype = None
        L.cxxattn_linattn_fwd_noalloc.argtypes = [C.POINTER(LinDesc)] + [vp] * 6 + [vp]
        L.cxxattn_linattn_noalloc_capacity.restype = sz
        L.cxxattn_linattn_noalloc_capacity.argtypes = []
        L.cxxattn_host_plan_create.argtypes = [C.POINTER(vp), C.POINTER(MhaDesc), i32]
        L.cxxattn_host_plan_destroy.argtypes = [vp]
        L.cxxattn_host_plan_destroy.restype = None
        L.cxxattn_mha_fwd_bwd_host.argtypes = [vp] * 9
        L.cxxattn_selftest_umma.argtypes = [i32, vp, vp, vp, vp]
        L.cxxattn_lin_host_plan_create.argtypes = [C.POINTER(vp), C.POINTER(LinDesc), i32]
        L.cxxattn_lin_host_plan_destroy.argtypes = [vp]
        L.cxxattn_lin_host_plan_destroy.restype = None
        L.cxxattn_linattn_fwd_bwd_host.argtypes = [vp] * 10
        L.cxxattn_set_option.argtypes = [i32, i32]
        L.cxxattn_get_option.argtypes = [i32, C.POINTER(i32)]
        L.cxxattn_selftest_wait_limit.argtypes = [C.c_uint64, vp]
        f32 = C.c_float
        L.cxxattn_adamw_step.argtypes = [vp, vp, vp, vp, sz, f32, f32, f32, f32, f32, f32, i32, vp, vp]
        L.cxxattn_adamw_step_mixed.argtypes = [vp, vp, vp, vp, vp, sz, f32, f32, f32, f32, f32, f32, i32, vp, vp]
        L.cxxattn_adamw_step_exchange.argtypes = [vp, vp, vp, C.POINTER(vp), C.POINTER(vp), i32, i32, i32, sz, sz,
                                                  f32, f32, f32, f32, f32, f32, i32, vp, vp]
        L.cxxattn_colsum_workspace_bytes.argtypes = [sz]
        L.cxxattn_colsum_workspace_bytes.restype = sz
        L.cxxattn_colsum.argtypes = [vp, i32, vp, sz, sz, vp, sz, vp]
        L.cxxattn_layernorm_bwd_workspace_bytes.argtypes = [sz]
        L.cxxattn_layernorm_bwd_workspace_bytes.restype = sz
        L.cxxattn_layernorm_bwd.argtypes = [vp] * 8 + [sz, sz, i32, vp, sz, vp]
        L.cxxattn_peer_alloc.argtypes = [sz, C.POINTER(vp)]
        L.cxxattn_peer_free.argtypes = [vp]
        L.cxxattn_peer_export.argtypes = [vp, C.c_char_p]
        L.cxxattn_peer_open.argtypes = [C.c_char_p, C.POINTER(vp)]
        L.cxxattn_peer_close.argtypes = [vp]
        _lib = L
    return _lib


def strerror(code):
    return lib().cxxattn_strerror(int(code)).decode()


def check(code, what):
    if code != 0:
        raise CxxAttnError(code, what)


# ---------------------------------------------------------------------------------------------
# torch plumbing: device pointers, the current stream, cached workspaces
# ---------------------------------------------------------------------------------------------

def _ptr(t, strided=False):
    """Device address of a tensor.  `strided`: the caller describes the layout through the
    descriptor's strides (a view into a larger tensor), so the view need not be contiguous."""
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("cxxattn kernels take CUDA tensors; there is no CPU path")
    if not strided and not t.is_contiguous():
        raise ValueError("tensor must be contiguous")
    return t.data_ptr()


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


_ws_cache = {}


def workspace(nbytes, device):
    """A cached device byte buffer of at least nbytes (grown on demand, one per device)."""
    import torch
    key = str(device)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


def _dtype_code(t):
    import torch
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise ValueError(f"unsupported dtype {t.dtype}")


def _dtype_code_of(dtype):
    import torch
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise ValueError(f"unsupported dtype {dtype}")


def mha_desc(B, S, H, Dh, dtype=F32, strides=None):
    sb, ss, sh = strides if strides else (0, 0, 0)
    return MhaDesc(B, S, H, Dh, sb, ss, sh, dtype, 0)


def lin_desc(B, S, D, E, dtype=F32, feature_map=MAP_ELU1, eps_in_den=0, ld_qk=0):
    return LinDesc(B, S, D, E, dtype, feature_map, eps_in_den, ld_qk)


# ---------------------------------------------------------------------------------------------
# thin C-ABI callers
# ---------------------------------------------------------------------------------------------

def mha_fwd(Q, K, V, O, B, S, H, Dh, lse=None, strides=None):
    d = mha_desc(B, S, H, Dh, _dtype_code(Q), strides)
    v = strides is not None
    check(lib().cxxattn_mha_fwd(C.byref(d), _ptr(Q, v), _ptr(K, v), _ptr(V, v), _ptr(O, v), _ptr(lse), _stream()),
          "cxxattn_mha_fwd")


def mha_bwd(Q, K, V, O, dO, dQ, dK, dV, B, S, H, Dh, lse=None, strides=None):
    d = mha_desc(B, S, H, Dh, _dtype_code(Q), strides)
    n = lib().cxxattn_mha_bwd_workspace_bytes(C.byref(d), int(lse is not None))
    ws = workspace(n, Q.device)
    v = strides is not None
    check(lib().cxxattn_mha_bwd(C.byref(d), _ptr(Q, v), _ptr(K, v), _ptr(V, v), _ptr(O, v), _ptr(dO, v), _ptr(lse),
                                _ptr(dQ, v), _ptr(dK, v), _ptr(dV, v), ws.data_ptr(), ws.numel(), _stream()),
          "cxxattn_mha_bwd")


def _lin_ws(d, device):
    n = lib().cxxattn_linattn_workspace_bytes(C.byref(d))
    return workspace(n, device)


def linattn_fwd(Q, K, V, O, den, z_cache, B, S, D, E, feature_map, eps_in_den):
    d = lin_desc(B, S, D, E, _dtype_code(Q), feature_map, eps_in_den)
    ws = _lin_ws(d, Q.device)
    check(lib().cxxattn_linattn_fwd(C.byref(d), _ptr(Q), _ptr(K), _ptr(V), _ptr(O), _ptr(den),
                                    _ptr(z_cache), ws.data_ptr(), ws.numel(), _stream()),
          "cxxattn_linattn_fwd")


def linattn_bwd_step1(O, dO, den, dnum, dden, N, E):
    check(lib().cxxattn_linattn_bwd_step1(_ptr(O), _ptr(dO), _ptr(den), _ptr(dnum), _ptr(dden), N, E,
                                          _stream()), "cxxattn_linattn_bwd_step1")


def linattn_bwd_dq(K, V, dnum, dden, z_cache, Q, dQ, B, S, D, E, feature_map, eps_in_den):
    d = lin_desc(B, S, D, E, F32, feature_map, eps_in_den)
    ws = _lin_ws(d, K.device)
    check(lib().cxxattn_linattn_bwd_dq(C.byref(d), _ptr(K), _ptr(V), _ptr(dnum), _ptr(dden),
                                       _ptr(z_cache), _ptr(Q), _ptr(dQ), ws.data_ptr(), ws.numel(),
                                       _stream()), "cxxattn_linattn_bwd_dq")


def linattn_bwd_dkdv(Q, K, V, dnum, dden, dK, dV, B, S, D, E, feature_map, eps_in_den):
    d = lin_desc(B, S, D, E, F32, feature_map, eps_in_den)
    ws = _lin_ws(d, K.device)
    check(lib().cxxattn_linattn_bwd_dkdv(C.byref(d), _ptr(Q), _ptr(K), _ptr(V), _ptr(dnum), _ptr(dden),
                                         _ptr(dK), _ptr(dV), ws.data_ptr(), ws.numel(), _stream()),
          "cxxattn_linattn_bwd_dkdv")


def linattn_bwd(Q, K, V, O, dO, den, dQ, dK, dV, B, S, D, E, feature_map, eps_in_den):
    d = lin_desc(B, S, D, E, _dtype_code(Q), feature_map, eps_in_den)
    ws = _lin_ws(d, Q.device)
    check(lib().cxxattn_linattn_bwd(C.byref(d), _ptr(Q), _ptr(K), _ptr(V), _ptr(O), _ptr(dO), _ptr(den),
                                    _ptr(dQ), _ptr(dK), _ptr(dV), ws.data_ptr(), ws.numel(), _stream()),
          "cxxattn_linattn_bwd")


class HostPlan:
    """Owner of the device staging buffers behind cxxattn_mha_fwd_bwd_host (host tensors in,
    host tensors out; torch CPU tensors, ideally pinned)."""

    def __init__(self, B, S, H, Dh, dtype, batch_per_chunk):
        self.handle = C.c_void_p()
        d = mha_desc(B, S, H, Dh, dtype)
        check(lib().cxxattn_host_plan_create(C.byref(self.handle), C.byref(d), batch_per_chunk),
              "cxxattn_host_plan_create")

    def fwd_bwd(self, Q, K, V, dO, O, dQ, dK, dV):
        ptrs = [t.data_ptr() for t in (Q, K, V, dO, O, dQ, dK, dV)]
        check(lib().cxxattn_mha_fwd_bwd_host(self.handle, *ptrs), "cxxattn_mha_fwd_bwd_host")

    def close(self):
        if self.handle:
            lib().cxxattn_host_plan_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LinHostPlan:
    """Owner of the device staging buffers behind cxxattn_linattn_fwd_bwd_host (host tensors in,
    host tensors out; heads folded into the B units)."""

    def __init__(self, B, S, D, E, dtype, units_per_chunk, feature_map=MAP_ELU1, eps_in_den=0):
        self.handle = C.c_void_p()
        d = lin_desc(B, S, D, E, dtype, feature_map, eps_in_den)
        check(lib().cxxattn_lin_host_plan_create(C.byref(self.handle), C.byref(d), units_per_chunk),
              "cxxattn_lin_host_plan_create")

    def fwd_bwd(self, Q, K, V, dO, O, den, dQ, dK, dV):
        ptrs = [t.data_ptr() for t in (Q, K, V, dO, O, den, dQ, dK, dV)]
        check(lib().cxxattn_linattn_fwd_bwd_host(self.handle, *ptrs), "cxxattn_linattn_fwd_bwd_host")

    def close(self):
        if self.handle:
            lib().cxxattn_lin_host_plan_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def set_option(option, value):
    """Process-wide schedule switch (OPT_*); see cxxattn_set_option."""
    check(lib().cxxattn_set_option(int(option), int(value)), "cxxattn_set_option")


def get_option(option):
    v = C.c_int(0)
    check(lib().cxxattn_get_option(int(option), C.byref(v)), "cxxattn_get_option")
    return v.value


class forced_option:
    """with forced_option(OPT_x, v): ... sets the option and puts the old value back."""

    def __init__(self, option, value):
        self.option, self.value = option, value

    def __enter__(self):
        self.old = get_option(self.option)
        set_option(self.option, self.value)

    def __exit__(self, *exc):
        set_option(self.option, self.old)


def adamw_step(param, grad, m, v, step, lr, beta1=0.9, beta2=0.999, weight_decay=0.01, eps=1e-8, grad_scale=1.0,
               grad_norm_sq=None, param_copy=None):
    """Fused mean-of-ranks + AdamW + squared gradient norm over flat buffers: fp32 gradient
    (cxxattn_adamw_step), or bf16 gradient with a bf16 copy of the parameters written in the same pass
    (cxxattn_adamw_step_mixed; param_copy required)."""
    import torch
    if grad.dtype == torch.bfloat16:
        check(lib().cxxattn_adamw_step_mixed(_ptr(param), _ptr(grad), _ptr(m), _ptr(v), _ptr(param_copy), param.numel(),
                                             float(grad_scale), float(lr), float(beta1), float(beta2),
                                             float(weight_decay), float(eps), int(step), _ptr(grad_norm_sq), _stream()),
              "cxxattn_adamw_step_mixed")
        return
    check(lib().cxxattn_adamw_step(_ptr(param), _ptr(grad), _ptr(m), _ptr(v), param.numel(), float(grad_scale),
                                   float(lr), float(beta1), float(beta2), float(weight_decay), float(eps), int(step),
                                   _ptr(grad_norm_sq), _stream()), "cxxattn_adamw_step")


def adamw_step_exchange(param_shard, m_shard, v_shard, grad_ptrs, param_ptrs, dtype, rank, lo, step, lr, beta1=0.9,
                        beta2=0.999, weight_decay=0.01, eps=1e-8, grad_scale=1.0, grad_norm_sq=None):
    """Gradient exchange + AdamW of one data-parallel rank over peer memory (cxxattn_adamw_step_exchange).
    grad_ptrs / param_ptrs: device addresses (ints), one per rank, of the ranks' whole gradient and
    parameter buffers of torch dtype `dtype` as this rank's GPU sees them; the rank owns elements
    [lo, lo + param_shard.numel())."""
    world = len(grad_ptrs)
    arr = C.c_void_p * world
    check(lib().cxxattn_adamw_step_exchange(_ptr(param_shard), _ptr(m_shard), _ptr(v_shard), arr(*grad_ptrs),
                                            arr(*param_ptrs), _dtype_code_of(dtype), world, int(rank), int(lo),
                                            param_shard.numel(), float(grad_scale), float(lr), float(beta1),
                                            float(beta2), float(weight_decay), float(eps), int(step),
                                            _ptr(grad_norm_sq), _stream()), "cxxattn_adamw_step_exchange")


def colsum_workspace_bytes(cols):
    return int(lib().cxxattn_colsum_workspace_bytes(int(cols)))


def colsum(X, out, workspace):
    """out[c] = sum over the rows of the 2-D tensor X (cxxattn_colsum); `workspace`: a uint8 tensor of at least
    colsum_workspace_bytes(cols) bytes that was zero before its first use."""
    rows, cols = X.shape
    check(lib().cxxattn_colsum(_ptr(X), _dtype_code(X), _ptr(out), rows, cols, _ptr(workspace), workspace.numel(),
                               _stream()), "cxxattn_colsum")


def layernorm_bwd_workspace_bytes(cols):
    return int(lib().cxxattn_layernorm_bwd_workspace_bytes(int(cols)))


def layernorm_bwd(dy, x, gamma, mean, rstd, dx, dgamma, dbeta, workspace):
    """LayerNorm backward (cxxattn_layernorm_bwd): dy, x, dx 2-D, gamma / dgamma / dbeta of the row width, all of one
    dtype; mean, rstd fp32 per row; `workspace` a uint8 tensor that was zero before its first use."""
    rows, cols = x.shape
    check(lib().cxxattn_layernorm_bwd(_ptr(dy), _ptr(x), _ptr(gamma), _ptr(mean), _ptr(rstd), _ptr(dx), _ptr(dgamma),
                                      _ptr(dbeta), rows, cols, _dtype_code(x), _ptr(workspace), workspace.numel(),
                                      _stream()), "cxxattn_layernorm_bwd")


class PeerBuffer:
    """A device buffer other processes' GPUs of this machine can map (cxxattn_peer_*).  `tensor` is a
    flat torch view of it; `handle()` is what another process passes to `PeerBuffer.open`."""

    def __init__(self, numel, dtype, device):
        import torch
        self.numel, self.dtype, self.device = int(numel), dtype, torch.device(device)
        self.itemsize = torch.empty(0, dtype=dtype).element_size()
        self.ptr, self.owned = C.c_void_p(), True
        with torch.cuda.device(self.device):
            check(lib().cxxattn_peer_alloc(max(1, self.numel) * self.itemsize, C.byref(self.ptr)), "cxxattn_peer_alloc")
        self.tensor = self._view()
        self.tensor.zero_()

    def _view(self):
        import torch
        raw = torch.as_tensor(_CudaArray(self.ptr.value, self.numel * self.itemsize, self), device=self.device)
        return raw.view(self.dtype)

    def handle(self):
        buf = C.create_string_buffer(64)
        check(lib().cxxattn_peer_export(self.ptr, buf), "cxxattn_peer_export")
        return buf.raw

    @classmethod
    def open(cls, handle, numel, dtype, device):
        """Maps a buffer another process exported; only the address is used (`ptr.value`)."""
        import torch
        self = cls.__new__(cls)
        self.numel, self.dtype, self.device = int(numel), dtype, torch.device(device)
        self.itemsize = torch.empty(0, dtype=dtype).element_size()
        self.ptr, self.owned, self.tensor = C.c_void_p(), False, None
        with torch.cuda.device(self.device):
            check(lib().cxxattn_peer_open(C.create_string_buffer(handle, 64), C.byref(self.ptr)), "cxxattn_peer_open")
        return self

    def close(self):
        if self.ptr and self.ptr.value:
            import torch
            with torch.cuda.device(self.device):
                (lib().cxxattn_peer_free if self.owned else lib().cxxattn_peer_close)(self.ptr)
            self.ptr = C.c_void_p()


class _CudaArray:
    """A byte range of device memory for torch.as_tensor (the CUDA array interface); keeps its owner alive."""

    def __init__(self, ptr, nbytes, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def selftest_wait_limit(limit_ns):
    check(lib().cxxattn_selftest_wait_limit(int(limit_ns), _stream()), "cxxattn_selftest_wait_limit")


def set_timing_events(start, stop):
    """torch.cuda.Event objects (enable_timing=True, already recorded once so that they exist) or
    None, None: recorded around the main backward kernel by the following mha_bwd calls."""
    lib().cxxattn_set_timing_events(start.cuda_event if start is not None else None,
                                    stop.cuda_event if stop is not None else None)


def sync_status():
    """Synchronises the current stream and raises if a tensor-core kernel gave up a bounded wait."""
    rc = lib().cxxattn_sync_status(_stream())
    if rc != 0:
        raise CxxAttnError(rc, "cxxattn_sync_status (wait site %d)" % lib().cxxattn_last_timeout_site())


def cast(src, dst):
    """dst = src converted between float32 and bfloat16 (dense tensors of equal element count)."""
    check(lib().cxxattn_cast(_ptr(src), _dtype_code(src), _ptr(dst), _dtype_code(dst), src.numel(), _stream()),
          "cxxattn_cast")


def rope_cast(src, dst, B, S, D, head_dim, sign=1.0):
    """dst = rotary embedding of src ([B*S, D], sign=+1 forward, -1 backward), converting between
    float32 and bfloat16 in the same pass (two_stage_gpt.hpp:102,113,160,174 with the conversion
    that the tensor-core kernels need)."""
    check(lib().cxxattn_rope_cast(_ptr(src), _dtype_code(src), _ptr(dst), _dtype_code(dst), B, S, D, head_dim,
                                  float(sign), _stream()), "cxxattn_rope_cast")


def rope_cast_pair(src0, src1, dst0, dst1, B, S, D, head_dim, sign=1.0):
    """rope_cast on two tensors of one shape and dtype pair in one launch (the reference's rope_fwd(Q, K, ...))."""
    check(lib().cxxattn_rope_cast_pair(_ptr(src0), _ptr(src1), _dtype_code(src0), _ptr(dst0), _ptr(dst1), _dtype_code(dst0),
                                       B, S, D, head_dim, float(sign), _stream()), "cxxattn_rope_cast_pair")


def linattn_decode_step(q, k, v, state_S, state_z, o, den, B, D, E, feature_map=MAP_ELU1, eps_in_den=0):
    """One new token per unit through the linear stage; state_S [B, D, E] and state_z [B, D] are
    updated in place (zero before the first token)."""
    d = lin_desc(B, 1, D, E, F32, feature_map, eps_in_den)
    check(lib().cxxattn_linattn_decode_step(C.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(state_S), _ptr(state_z),
                                            _ptr(o), _ptr(den), _stream()), "cxxattn_linattn_decode_step")


def mha_decode_step(q, k, v, K_cache, V_cache, pos, o, B, capacity, H, Dh):
    """One new token per batch item through the softmax stage; k, v are appended to the caches
    [B, capacity, H*Dh] at row pos."""
    d = mha_desc(B, capacity, H, Dh, F32)
    n = lib().cxxattn_mha_decode_workspace_bytes(C.byref(d))
    ws = workspace(n, q.device) if n else None
    check(lib().cxxattn_mha_decode_step(C.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(K_cache), _ptr(V_cache), int(pos),
                                        _ptr(o), _ptr(ws), n, _stream()), "cxxattn_mha_decode_step")


def selftest_umma(mode, A, B, D):
    check(lib().cxxattn_selftest_umma(mode, _ptr(A), _ptr(B), _ptr(D), _stream()), "cxxattn_selftest_umma")


# ---------------------------------------------------------------------------------------------
# the reference's operator interface, by name
# ---------------------------------------------------------------------------------------------

class two_stage_cuda:
    """namespace two_stage_cuda (src/TwoStage/two_stage_cuda_kernels.cuh:18-85)."""

    @staticmethod
    def fused_mha_fwd(Q, K, V, O, B, S, H, Dh):
        mha_fwd(Q, K, V, O, B, S, H, Dh)

    @staticmethod
    def fused_mha_bwd(Q, K, V, O, dO, dQ, dK, dV, B, S, H, Dh):
        mha_bwd(Q, K, V, O, dO, dQ, dK, dV, B, S, H, Dh)

    @staticmethod
    def kernel_attn_fwd(Q, K, V, O, den_cache, z_cache, S_buf, z_buf, B, S, D, E):
        # S_buf / z_buf are the reference's serial-scan scratch; the chunked scan does not use them.
        linattn_fwd(Q, K, V, O, den_cache, z_cache, B, S, D, E, MAP_ELU1, 0)

    @staticmethod
    def kernel_attn_bwd_step1(O, dO, den_cache, dnum, dden, N, E):
        linattn_bwd_step1(O, dO, den_cache, dnum, dden, N, E)

    @staticmethod
    def kernel_attn_bwd_dQ(K, V, dnum, dden, z_cache, Q, dQ, S_buf, B, S, D, E):
        linattn_bwd_dq(K, V, dnum, dden, z_cache, Q, dQ, B, S, D, E, MAP_ELU1, 0)

    @staticmethod
    def kernel_attn_bwd_dKdV(Q, K, V, dnum, dden, dK, dV, B, S, D, E):
        linattn_bwd_dkdv(Q, K, V, dnum, dden, dK, dV, B, S, D, E, MAP_ELU1, 0)

    @staticmethod
    def rope_fwd(Q, K, B, S, D, head_dim):
        check(lib().cxxattn_rope(_ptr(Q), _ptr(K), B, S, D, head_dim, 1.0, _stream()), "cxxattn_rope")

    @staticmethod
    def rope_bwd(dQ, dK, B, S, D, head_dim):
        check(lib().cxxattn_rope(_ptr(dQ), _ptr(dK), B, S, D, head_dim, -1.0, _stream()), "cxxattn_rope")

    @staticmethod
    def gelu_exact(A, Cout):
        check(lib().cxxattn_gelu_exact(_ptr(A), _ptr(Cout), A.numel(), 0, _stream()), "cxxattn_gelu_exact")

    @staticmethod
    def gelu_exact_deriv(A, Cout):
        check(lib().cxxattn_gelu_exact(_ptr(A), _ptr(Cout), A.numel(), 1, _stream()), "cxxattn_gelu_exact")


class linear_cuda:
    """namespace linear_cuda (src/LinearAttention/linear_cuda_kernels.cuh:11-46)."""

    @staticmethod
    def causal_linear_attention_fwd(Q_phi, K_phi, V, O, den_cache, z_cache, S_buf, z_buf, B, S, D, E):
        linattn_fwd(Q_phi, K_phi, V, O, den_cache, z_cache, B, S, D, E, MAP_NONE, 1)

    @staticmethod
    def causal_linear_attention_bwd_step1(O, dO, den_cache, dnum, dden, N, E):
        linattn_bwd_step1(O, dO, den_cache, dnum, dden, N, E)

    @staticmethod
    def causal_linear_attention_bwd_dQ(K_phi, V, dnum, dden, z_cache, dQ_phi, S_buf, B, S, D, E):
        linattn_bwd_dq(K_phi, V, dnum, dden, z_cache, None, dQ_phi, B, S, D, E, MAP_NONE, 1)

    @staticmethod
    def causal_linear_attention_bwd_dKdV(Q_phi, K_phi, V, dnum, dden, dK_phi, dV, B, S, D, E):
        linattn_bwd_dkdv(Q_phi, K_phi, V, dnum, dden, dK_phi, dV, B, S, D, E, MAP_NONE, 1)

    @staticmethod
    def phi_elu_forward(x, phi, D, E):
        check(lib().cxxattn_phi_elu_fwd(_ptr(x), _ptr(phi), x.shape[0], D, E, _stream()), "cxxattn_phi_elu_fwd")

    @staticmethod
    def phi_elu_backward(dphi, x, dx, D, E):
        check(lib().cxxattn_phi_elu_bwd(_ptr(dphi), _ptr(x), _ptr(dx), dphi.shape[0], D, E, _stream()),
              "cxxattn_phi_elu_bwd")
