"""Regenerates the committed golden vectors from the reference checkout.

Run where the reference tree is available:
    python tests/golden/make_golden.py /path/to/deepstrix

Outputs (small, committed):
  mxfp4_selftest.npz   the reference's own known-answer vector for MXFP4 dequant:
      `expected` = the 256 f32 bit patterns of external/ds4-dump/quants_selftest_expected.inc
      (array expected_mxfp4), `blocks` = the 8 ggml blocks its generator builds
      (external/ds4-dump/quants_selftest.c:45-53,82-87,102-105: LCG bytes, seed 0x3333,
      scale bytes forced to 120..127)
  kernelpy_vectors.npz inputs and outputs of the reference's CPU oracle
      scripts/v41_oracle/kernel.py (dequant_fp4, q8_0_roundtrip, act_quant, fp4_act_quant, fp4_gemm),
      imported and executed unmodified under torch-CPU
"""
import importlib.util
import os
import re
import sys

import numpy as np


def lcg_bytes(seed: int, n: int) -> np.ndarray:
    state = seed & 0xFFFFFFFF
    out = np.empty(n, np.uint8)
    for i in range(n):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = state >> 24
    return out


def main(ref: str):
    here = os.path.dirname(os.path.abspath(__file__))
    inc = open(os.path.join(ref, "external/ds4-dump/quants_selftest_expected.inc")).read()
    body = inc[inc.index("expected_mxfp4[256]"):]
    body = body[body.index("{") + 1: body.index("}")]
    expected = np.array([int(x, 16) for x in re.findall(r"0x[0-9a-fA-F]+", body)], np.uint32)
    assert expected.size == 256
    blocks = lcg_bytes(0x3333, 8 * 17)
    for i in range(8):
        blocks[i * 17] = 120 + i
    np.savez(os.path.join(here, "mxfp4_selftest.npz"), expected=expected, blocks=blocks)

    import torch
    spec = importlib.util.spec_from_file_location("ref_kernel", os.path.join(ref, "scripts/v41_oracle/kernel.py"))
    k = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(k)
    rng = np.random.Generator(np.random.PCG64(0xD5EE))
    rows, K = 48, 512
    packed = rng.integers(0, 256, size=(rows, K // 2), dtype=np.uint8)
    scales = rng.integers(110, 136, size=(rows, K // 32), dtype=np.uint8)
    s_t = torch.from_numpy(scales).view(torch.float8_e8m0fnu)
    deq = k.dequant_fp4(torch.from_numpy(packed), s_t).numpy()
    x = rng.standard_normal((5, K)).astype(np.float32) * 3.0
    torch.set_default_dtype(torch.float32)
    xq, xs = k.act_quant(torch.from_numpy(x), block_size=32, scale_fmt="ue8m0")
    gemm = k.fp4_gemm(xq, xs, torch.from_numpy(packed), s_t).float().numpy()
    xq_f = (xq.float().view(5, K // 32, 32) * xs.float().unsqueeze(-1)).view(5, K).numpy()
    # MXFP4 activation terms: the reference's FP4 fake-quant (fp4_act_quant, block 32, E8M0 scales) applied to x,
    # then to what it left over, three times; terms[i] is the dequantised i-th term
    res = torch.from_numpy(x).clone()
    terms = []
    for _ in range(3):
        y, _s = k.fp4_act_quant(res, block_size=32)
        terms.append(y.float().numpy().copy())
        res = res - y.float()
    w = rng.standard_normal((8, 64)).astype(np.float32)
    q8rt = k.q8_0_roundtrip(torch.from_numpy(w)).numpy()
    np.savez(os.path.join(here, "kernelpy_vectors.npz"), packed=packed, scales=scales, dequant=deq, x=x,
             x_fp8_dequant=xq_f, fp4_gemm=gemm, q8_in=w, q8_roundtrip=q8rt, x_fp4_terms=np.stack(terms))
    print("wrote", sorted(os.listdir(here)))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a checkout of the deepstrix repository>")
    main(sys.argv[1])
