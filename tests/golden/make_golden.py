"""Produces the golden fixtures of this directory by running the REFERENCE itself.

Needs a B200 and ``oracle/_ref/libtcec_ref.so`` (the reference's headers and its
batched example kernel compiled for sm_100a by ``oracle/Makefile``).  Run from the
repository root:

    python tests/golden/make_golden.py <output directory>

and copy the ``.npz`` files it writes into ``tests/golden/``.  Inputs are seeded;
they are stored next to the outputs so the tests do not depend on a generator's
bit stream staying stable.
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from oracle import ref  # noqa: E402


def split_inputs() -> np.ndarray:
    rng = np.random.default_rng(11)
    special = np.array(
        [0.0, -0.0, 1.0, -1.0, 0.5, 1.0 / 3.0, 65504.0, 65519.99, 65520.0, 70000.0, -70000.0, 1e-8, 6e-8, 5.96e-8,
         2.98e-8, 2.9802322e-8, 6.1035156e-5, 6.0975552e-5, 1e-5, 3e-5, 1.0009766, 1.0004883, 1.0014648, 2049.0,
         2051.0, 4097.0, 0.1, 0.2, 0.3, 1e4, 3.1415927, 2.7182817, 1e-3, 1e-30, 1e30, 3.4028235e38,
         1.17549435e-38, 1.0 + 2.0 ** -11, 1.0 + 2.0 ** -11 + 2.0 ** -23, 1.0 + 3 * 2.0 ** -11,
         1.0 + 2.0 ** -12, 1.0 + 2.0 ** -13], dtype=np.float32)
    uni = rng.uniform(-1, 1, 1024).astype(np.float32)
    wide = (rng.choice([-1.0, 1.0], 1024) * rng.uniform(1, 2, 1024) * np.exp2(rng.integers(-30, 18, 1024))).astype(
        np.float32)
    # exact ties for tf32 (bit 12 set, lower bits clear) and for fp16 (bit 12 set in the 13 dropped bits)
    base = rng.uniform(1, 2, 256).astype(np.float32).view(np.uint32)
    ties = ((base & np.uint32(0xFFFFE000)) | np.uint32(0x1000)).view(np.float32)
    return np.concatenate([special, uni, wide, ties, -ties]).astype(np.float32)


def main(outdir: str) -> None:
    os.makedirs(outdir, exist_ok=True)
    dev = torch.device("cuda:0")
    # ---- split: bit-exact pin of the hi / lo arithmetic
    x = split_inputs()
    xd = torch.from_numpy(x).to(dev)
    out = {"x": x}
    for name, tf32 in (("fp16", False), ("tf32", True)):
        hi, lo = ref.split(xd, tf32)
        out[f"hi_{name}"] = hi.cpu().numpy()
        out[f"lo_{name}"] = lo.cpu().numpy()
    np.savez_compressed(os.path.join(outdir, "ref_split.npz"), **out)

    # ---- one warp, 32x32x32 (the reference's own unit-test shape, test/tcec/mma.cu:192)
    rng = np.random.default_rng(1)
    a = rng.uniform(-1, 1, (32, 32)).astype(np.float32)
    b = rng.uniform(-1, 1, (32, 32)).astype(np.float32)
    c = rng.uniform(-1, 1, (32, 32)).astype(np.float32)
    ad, bd, cd = (torch.from_numpy(t).to(dev) for t in (a, b, c))
    out = {"a": a, "b": b, "c": c}
    for tf32 in (False, True):
        for op_wmma in (False, True):
            for ec in (False, True):
                for with_c in (False, True):
                    for rz in (False, True):
                        key = f"d_{'tf32' if tf32 else 'fp16'}_{'wmma' if op_wmma else 'mma'}_{'ec' if ec else 'noec'}" \
                              f"_{'abcd' if with_c else 'abd'}_{'rz' if rz else 'default'}"
                        d = ref.warp_mma(ad, bd, cd if with_c else None, tf32, op_wmma, ec, rz)
                        out[key] = d.cpu().numpy()
    np.savez_compressed(os.path.join(outdir, "ref_warp_mma.npz"), **out)

    # ---- the reference's batched tile pipeline (test/tcec/batch_gemm.cu:261-386)
    rng = np.random.default_rng(4)
    a = rng.standard_normal((2, 128, 160)).astype(np.float32)
    b = rng.standard_normal((2, 160, 128)).astype(np.float32)
    ad, bd = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
    out = {"a": a, "b": b}
    for tf32 in (False, True):
        cref = ref.bgemm(ad, bd, tf32=tf32, per=1)
        out[f"c_{'tf32' if tf32 else 'fp16'}"] = cref.contiguous().cpu().numpy()
    # its own deterministic inputs, A[j] = j / k, B[j] = j / n (test/tcec/batch_gemm.cu:507-513), small size
    m = n = 128
    k = 64
    a2 = (np.arange(m * k, dtype=np.float32) / np.float32(k)).reshape(1, m, k)
    b2_colmajor = (np.arange(k * n, dtype=np.float32) / np.float32(n)).reshape(1, n, k)  # ldb = k, column-major
    b2 = np.ascontiguousarray(b2_colmajor.transpose(0, 2, 1))
    cref = ref.bgemm(torch.from_numpy(a2).to(dev), torch.from_numpy(b2).to(dev), tf32=False, per=1)
    out["a_iota"], out["b_iota"], out["c_iota_fp16"] = a2, b2, cref.contiguous().cpu().numpy()
    np.savez_compressed(os.path.join(outdir, "ref_bgemm.npz"), **out)
    print("wrote", sorted(os.listdir(outdir)))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "golden_out")
