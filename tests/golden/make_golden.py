"""Generates tests/golden/*.npz from the REFERENCE's own CPU functions (src/TwoStage/
kernel_test.cpp compiled where it lies, see oracle/ref_wrap.cpp).  Run in a container that has
the reference tree mounted:

    python tests/golden/make_golden.py

Contents
  kernel_test_blocks.npz  for each of the six attention blocks of the reference kernel test
      (same std::mt19937(1234) input stream): the reference outputs.  Small blocks are stored
      whole; the three large ones as every 61st element plus float64 sum / sum of |x|.
      Also the first 64 draws of the input stream, which pins the generator itself.
  seeded_cases.npz        reference outputs for the seeded normal inputs used by the GPU tests
      at the small baseline configurations (softmax B=8,S=64,H=4,Dh=32; ELU+1 B=32,S=64,D=E=32).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from conftest import KT_BLOCKS, kt_block_inputs, seeded_normal  # noqa: E402

STRIDE = 61


def pack(out, name, a, whole):
    a = np.asarray(a, np.float32).ravel()
    if whole:
        out[name] = a
    else:
        out[name + "__sub"] = a[::STRIDE].copy()
        out[name + "__sum"] = np.array([a.astype(np.float64).sum(), np.abs(a.astype(np.float64)).sum()])


def main():
    ref = oracle.Reference()
    out = {"frand_head": ref.frand(64, 0)}
    for i, (kind, d) in enumerate(KT_BLOCKS):
        _, _, (Q, K, V, dO) = kt_block_inputs(ref.frand, i)
        whole = Q.size <= 4096
        if kind == "mha":
            O = ref.mha_fwd(Q, K, V, **d)
            dQ, dK, dV = ref.mha_bwd(Q, K, V, O, dO, **d)
            names = dict(O=O, dQ=dQ, dK=dK, dV=dV)
        else:
            O, den = ref.kernel_attn_fwd(Q, K, V, **d)
            dQ, dK, dV = ref.kernel_attn_bwd(Q, K, V, O, dO, den, **d)
            names = dict(O=O, den=den, dQ=dQ, dK=dK, dV=dV)
        for k, v in names.items():
            pack(out, f"b{i}_{k}", v, whole)
    np.savez_compressed(os.path.join(HERE, "kernel_test_blocks.npz"), **out)

    out = {}
    B, S, H, Dh = 8, 64, 4, 32
    Q, K, V, dO = seeded_normal(0, [(B * S, H * Dh)] * 4)
    O = ref.mha_fwd(Q, K, V, B, S, H, Dh)
    dQ, dK, dV = ref.mha_bwd(Q, K, V, O, dO, B, S, H, Dh)
    for k, v in dict(O=O, dQ=dQ, dK=dK, dV=dV).items():
        pack(out, "cfg1_" + k, v, False)
    B, S, D, E = 32, 64, 32, 32
    Q, K, V, dO = seeded_normal(1, [(B * S, D), (B * S, D), (B * S, E), (B * S, E)])
    O, den = ref.kernel_attn_fwd(Q, K, V, B, S, D, E)
    dQ, dK, dV = ref.kernel_attn_bwd(Q, K, V, O, dO, den, B, S, D, E)
    for k, v in dict(O=O, den=den, dQ=dQ, dK=dK, dV=dV).items():
        pack(out, "cfg2_" + k, v, False)
    np.savez_compressed(os.path.join(HERE, "seeded_cases.npz"), **out)
    for f in ("kernel_test_blocks.npz", "seeded_cases.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
