"""Generates the committed golden fixtures of this directory.  Run in the build container:

    python tests/golden/make_golden.py /path/to/reference        (or REFERENCE_ROOT=/path/to/reference)

1. ref_gen_data.npz - inputs and goldens produced by the reference's own data generators, imported from the
   reference tree (tests/ut/op_kernel/mat_mul/matmul_data/gen_data.py and
   tests/ut/op_kernel/quant_batch_matmul/qbmm_data/gen_data.py), with numpy's global generator seeded so the run is
   repeatable.  They pin the "golden style" the oracle adopts: up-cast to float32, np.matmul, scale, cast.
   ref_gen_kernels.npz holds further outputs of the same generators at tile-kernel shapes (A8W8 and fp16 matmul).
2. narrow_float_casts.npz - float32 inputs with the E4M3 / E2M1 codes ml_dtypes assigns them (after the explicit
   clamp that turns its NaN-on-overflow into saturation) and torch's E8M0 encoding of powers of two: independent
   implementations of the public element formats.

micro_vectors.json in this directory is hand-derived and is not produced by this script.
"""
import importlib.util
import os
import sys
import tempfile

import numpy as np


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT")
    if not ref:
        sys.exit("usage: make_golden.py /path/to/reference")
    here = os.path.dirname(os.path.abspath(__file__))
    out = {}
    mm = _load(os.path.join(ref, "tests/ut/op_kernel/mat_mul/matmul_data/gen_data.py"), "ref_mm_gen")
    qb = _load(os.path.join(ref, "tests/ut/op_kernel/quant_batch_matmul/qbmm_data/gen_data.py"), "ref_qbmm_gen")
    with tempfile.TemporaryDirectory() as tmp:
        np.random.seed(20260101)
        a, b, g = mm.gen_matmul_data(32, 48, 64, "float32", tmp)
        out.update(mm_f32_a=a, mm_f32_b=b, mm_f32_golden=g)
        np.random.seed(20260102)
        a, b, g = mm.gen_matmul_data(16, 16, 16, "float16", tmp)
        out.update(mm_f16_a=a, mm_f16_b=b, mm_f16_golden=g)
        np.random.seed(20260103)
        a, b, pts, sc, g = qb.gen_qbmm_data(16, 16, 16, tmp)
        out.update(qbmm_a=a, qbmm_b=b, qbmm_pertoken=pts, qbmm_scale=sc, qbmm_golden=g)
    np.savez_compressed(os.path.join(here, "ref_gen_data.npz"), **out)

    # ref_gen_kernels.npz - the same two generators at shapes a GPU tile kernel has to work for (ragged against the
    # 256 x 256 tiles and the 128-byte K blocks).  The A8W8 goldens are exact: the products are integers and K < 1024
    # keeps every float32 partial sum below 2^24, so any implementation of int32 accumulate + conversion + cast must
    # reproduce them bit for bit.  The fp16 golden depends on the summation order and pins results to a few ulp.
    big = {}
    with tempfile.TemporaryDirectory() as tmp:
        np.random.seed(20260104)
        a, b, pts, sc, g = qb.gen_qbmm_data(300, 264, 96, tmp)
        big.update(a8w8_300_a=a, a8w8_300_b=b, a8w8_300_golden=g)
        np.random.seed(20260105)
        a, b, pts, sc, g = qb.gen_qbmm_data(136, 264, 512, tmp)
        big.update(a8w8_136_a=a, a8w8_136_b=b, a8w8_136_golden=g)
        np.random.seed(20260106)
        a, b, g = mm.gen_matmul_data(136, 264, 160, "float16", tmp)
        big.update(mm_f16_136_a=a, mm_f16_136_b=b, mm_f16_136_golden=g)
    np.savez_compressed(os.path.join(here, "ref_gen_kernels.npz"), **big)

    import ml_dtypes
    import torch
    rng = np.random.default_rng(7)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * s for s in (1e-3, 1e-2, 0.3, 1, 20, 200)])
    x = np.concatenate([x, np.array([0.0, -0.0, 448, 449, 464, 465, 480, 1e6, -1e6, 2 ** -9, 2 ** -10, 3 * 2 ** -10,
                                     2 ** -6, 2 ** -6 - 2 ** -10], dtype=np.float32)])
    e4 = np.clip(x, -448, 448).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    y = np.concatenate([rng.standard_normal(2048).astype(np.float32) * s for s in (0.2, 1, 4)])
    y = np.concatenate([y, np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, 100.0, -0.25, -0.0],
                                    dtype=np.float32)])
    e2 = np.clip(y, -6, 6).astype(ml_dtypes.float4_e2m1fn).view(np.uint8) & 0xF
    p2 = np.exp2(np.arange(-127, 128, dtype=np.float64)).astype(np.float32)
    e8 = torch.from_numpy(p2).to(torch.float8_e8m0fnu).view(torch.uint8).numpy()
    np.savez_compressed(os.path.join(here, "narrow_float_casts.npz"), e4m3_in=x, e4m3_codes=e4, e2m1_in=y,
                        e2m1_codes=e2, e8m0_in=p2, e8m0_codes=e8)
    print("wrote", os.listdir(here))


if __name__ == "__main__":
    main()
