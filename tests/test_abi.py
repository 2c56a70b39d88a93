"""CPU checks of the drop-in boundary: the shared library loads, exports every symbol that the
headers under include/ declare, and rejects bad arguments with error codes before touching a device."""
import ctypes as C
import glob
import os
import re

from conftest import ROOT


def declared_symbols():
    names = set()
    for path in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        text = re.sub(r"/\*.*?\*/", "", open(path).read(), flags=re.S)
        names |= set(re.findall(r"\b(cxxattn_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.lib()
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared under include/ but not exported"
    assert set(pkg.SYMBOLS) <= set(names)


def test_version_and_strerror(pkg):
    assert b"sm_100a" in pkg.lib().cxxattn_version()
    assert pkg.strerror(0) == "ok"
    for code in range(-7, 0):
        assert pkg.strerror(code) not in ("ok", "unknown error")
    assert pkg.strerror(-99) == "unknown error"


def test_bad_arguments_are_rejected_without_a_device(pkg):
    lib = pkg.lib()
    d = pkg.mha_desc(2, 8, 2, 16)
    one = C.c_void_p(16)
    assert lib.cxxattn_mha_fwd(None, one, one, one, one, None, None) == -1
    assert lib.cxxattn_mha_fwd(C.byref(d), None, one, one, one, None, None) == -1
    bad = pkg.mha_desc(0, 8, 2, 16)
    assert lib.cxxattn_mha_fwd(C.byref(bad), one, one, one, one, None, None) == -1
    assert lib.cxxattn_mha_bwd_workspace_bytes(C.byref(bad), 0) == 0
    assert lib.cxxattn_mha_bwd_workspace_bytes(C.byref(d), 0) >= 2 * 2 * 2 * 8 * 4
    # backward without a workspace
    assert lib.cxxattn_mha_bwd(C.byref(d), one, one, one, one, one, None, one, one, one, None, 0, None) == -3
    # head dimension beyond 256 is unsupported, as in the reference (which aborts instead)
    big = pkg.mha_desc(1, 8, 1, 512)
    assert lib.cxxattn_mha_bwd(C.byref(big), one, one, one, one, one, None, one, one, one, one, 1 << 20, None) == -2
    ld = pkg.lin_desc(2, 8, 4, 4)
    assert lib.cxxattn_linattn_workspace_bytes(C.byref(ld)) > 0
    assert lib.cxxattn_linattn_fwd(C.byref(ld), one, one, one, one, one, None, None, 0, None) == -3
    badmap = pkg.lin_desc(2, 8, 4, 4, feature_map=7)
    assert lib.cxxattn_linattn_fwd(C.byref(badmap), one, one, one, one, one, None, one, 1 << 20, None) == -1
    assert lib.cxxattn_rope(None, None, 1, 1, 8, 8, 1.0, None) == -1
    assert lib.cxxattn_rope(one, one, 1, 1, 8, 3, 1.0, None) == -1
    assert lib.cxxattn_rope_cast(None, 0, one, 1, 1, 1, 8, 8, 1.0, None) == -1
    assert lib.cxxattn_rope_cast(one, 0, one, 1, 1, 1, 8, 6, 1.0, None) == -1   # head_dim % 4
    assert lib.cxxattn_rope_cast(one, 0, one, 1, 1, 1, 12, 8, 1.0, None) == -1  # D % head_dim
    assert lib.cxxattn_phi_elu_fwd(one, one, 4, 2, 4, None) == -1   # E > D
    dec = pkg.mha_desc(2, 16, 2, 8)
    assert lib.cxxattn_mha_decode_step(C.byref(dec), one, one, one, one, one, 16, one, None, 0, None) == -1  # pos >= S
    assert lib.cxxattn_mha_decode_step(C.byref(dec), one, one, one, None, one, 0, one, None, 0, None) == -1
    assert lib.cxxattn_mha_decode_workspace_bytes(C.byref(dec)) == 0   # 16 keys never need a split
    long = pkg.mha_desc(1, 8192, 2, 64)
    assert lib.cxxattn_mha_decode_workspace_bytes(C.byref(long)) > 0
    assert lib.cxxattn_mha_decode_step(C.byref(long), one, one, one, one, one, 8000, one, None, 0, None) == -3
    assert lib.cxxattn_linattn_decode_step(C.byref(ld), one, one, one, None, one, one, None, None) == -1
    assert lib.cxxattn_gelu_exact(one, one, 0, 0, None) == -1
    # decoding steps hold their descriptors to the same bounds as the other entry points
    huge = pkg.lin_desc(1 << 40, 8, 4, 4)
    assert lib.cxxattn_linattn_decode_step(C.byref(huge), one, one, one, one, one, one, None, None) == -1
    badeps = pkg.lin_desc(2, 8, 4, 4, eps_in_den=5)
    assert lib.cxxattn_linattn_decode_step(C.byref(badeps), one, one, one, one, one, one, None, None) == -1
    wide = pkg.mha_desc(1 << 20, 16, 1 << 20, 8)   # B*H beyond a 32-bit grid dimension
    assert lib.cxxattn_mha_decode_step(C.byref(wide), one, one, one, one, one, 0, one, None, 0, None) == -1
    # host plans: bad descriptors are refused before any allocation
    plan = C.c_void_p()
    assert lib.cxxattn_host_plan_create(C.byref(plan), C.byref(bad), 1) == -1
    assert lib.cxxattn_lin_host_plan_create(C.byref(plan), C.byref(pkg.lin_desc(0, 8, 4, 4)), 1) == -1
    assert lib.cxxattn_linattn_fwd_bwd_host(None, one, one, one, one, one, one, one, one, one) == -1
    assert lib.cxxattn_selftest_wait_limit(10, None) == -1            # below the smallest limit
    # exchange + optimiser step: rank set, shard bounds and pointers are checked before any launch
    two = (C.c_void_p * 2)(16, 32)
    f = [1.0, 1e-3, 0.9, 0.999, 0.01, 1e-8]
    ex = lib.cxxattn_adamw_step_exchange
    assert ex(one, one, one, two, two, pkg.BF16, 0, 0, 0, 8, *f, 1, None, None) == -1    # no ranks
    assert ex(one, one, one, two, two, pkg.BF16, 17, 0, 0, 8, *f, 1, None, None) == -1   # more than 16
    assert ex(one, one, one, two, two, pkg.BF16, 2, 2, 0, 8, *f, 1, None, None) == -1    # rank outside the set
    assert ex(one, one, one, two, two, pkg.BF16, 2, 0, 4, 8, *f, 1, None, None) == -1    # bf16 shard not on 8 elements
    assert ex(one, one, one, two, two, pkg.F32, 2, 0, 4, 6, *f, 1, None, None) == -1     # fp32 shard not on 4 elements
    assert ex(one, one, one, two, two, 9, 2, 0, 0, 8, *f, 1, None, None) == -1           # unknown dtype
    assert ex(one, one, one, two, two, pkg.BF16, 2, 0, 0, 8, *f, 0, None, None) == -1    # steps count from 1
    assert ex(None, one, one, two, two, pkg.BF16, 2, 0, 0, 8, *f, 1, None, None) == -1
    assert ex(one, one, one, (C.c_void_p * 2)(16, None), two, pkg.BF16, 2, 0, 0, 8, *f, 1, None, None) == -1
    assert ex(one, one, one, (C.c_void_p * 2)(16, 36), two, pkg.BF16, 2, 0, 0, 8, *f, 1, None, None) == -6  # alignment
    assert ex(None, None, None, two, two, pkg.BF16, 2, 1, 8, 0, *f, 1, None, None) == 0  # a rank that owns nothing
    # column sums
    assert lib.cxxattn_colsum_workspace_bytes(0) == 0 and lib.cxxattn_colsum_workspace_bytes(768) >= 768 * 4
    assert lib.cxxattn_colsum(None, pkg.BF16, one, 4, 8, one, 1 << 20, None) == -1
    assert lib.cxxattn_colsum(one, pkg.BF16, one, 0, 8, one, 1 << 20, None) == -1
    assert lib.cxxattn_colsum(one, 5, one, 4, 8, one, 1 << 20, None) == -1
    assert lib.cxxattn_colsum(one, pkg.BF16, one, 4, 12, one, 1 << 20, None) == -2     # bf16 rows in 16-byte vectors
    assert lib.cxxattn_colsum(one, pkg.BF16, one, 4, 8, one, 8, None) == -3            # workspace too small
    assert lib.cxxattn_colsum(one, pkg.BF16, one, 4, 8, None, 0, None) == -3
    # LayerNorm backward
    ln = lib.cxxattn_layernorm_bwd
    assert lib.cxxattn_layernorm_bwd_workspace_bytes(768) >= 2 * 768 * 4
    assert ln(None, one, one, one, one, one, one, one, 4, 8, pkg.BF16, one, 1 << 20, None) == -1
    assert ln(one, one, one, one, one, one, one, one, 4, 0, pkg.BF16, one, 1 << 20, None) == -1
    assert ln(one, one, one, one, one, one, one, one, 4, 12, pkg.BF16, one, 1 << 20, None) == -2
    assert ln(one, one, one, one, one, one, one, one, 4, 8, pkg.BF16, one, 8, None) == -3
    assert ln(one, one, one, one, one, C.c_void_p(20), one, one, 4, 8, pkg.BF16, one, 1 << 20, None) == -6
    p = C.c_void_p()
    assert lib.cxxattn_peer_alloc(0, C.byref(p)) == -1 and lib.cxxattn_peer_alloc(16, None) == -1
    assert lib.cxxattn_peer_export(None, C.create_string_buffer(64)) == -1
    assert lib.cxxattn_peer_open(None, C.byref(p)) == -1
    assert lib.cxxattn_peer_free(None) == 0 and lib.cxxattn_peer_close(None) == 0


def test_options_are_validated_and_readable(pkg):
    lib = pkg.lib()
    defaults = {pkg.OPT_FWD_LATE_WAIT: -1, pkg.OPT_BWD_PERSISTENT: -1, pkg.OPT_LIN_GROUPS: 0,
                pkg.OPT_LIN_SIDE_STREAM: 1}
    for opt, want in defaults.items():
        assert pkg.get_option(opt) == want
    assert lib.cxxattn_set_option(99, 0) == -1
    assert lib.cxxattn_set_option(pkg.OPT_FWD_LATE_WAIT, 2) == -1
    assert lib.cxxattn_set_option(pkg.OPT_LIN_GROUPS, -1) == -1
    assert lib.cxxattn_get_option(pkg.OPT_LIN_GROUPS, None) == -1
    with pkg.forced_option(pkg.OPT_LIN_GROUPS, 3):
        assert pkg.get_option(pkg.OPT_LIN_GROUPS) == 3
    assert pkg.get_option(pkg.OPT_LIN_GROUPS) == 0


def test_python_front_end_mirrors_reference_names(pkg):
    for n in ("fused_mha_fwd", "fused_mha_bwd", "kernel_attn_fwd", "kernel_attn_bwd_step1",
              "kernel_attn_bwd_dQ", "kernel_attn_bwd_dKdV", "rope_fwd", "rope_bwd", "gelu_exact",
              "gelu_exact_deriv"):
        assert callable(getattr(pkg.two_stage_cuda, n))
    for n in ("causal_linear_attention_fwd", "causal_linear_attention_bwd_step1",
              "causal_linear_attention_bwd_dQ", "causal_linear_attention_bwd_dKdV",
              "phi_elu_forward", "phi_elu_backward"):
        assert callable(getattr(pkg.linear_cuda, n))
