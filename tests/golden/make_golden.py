"""Generates the known-answer fixtures of this directory.

Run from the repository root:  python tests/golden/make_golden.py
Sources of truth: torch's float8_e4m3fn / bfloat16 CPU casts and ml_dtypes
(two independent implementations of OCP e4m3fn), plus exact integer
arithmetic for the tiny GEMMs.  The reference project has no golden vectors
for these paths, so these are self-generated.
"""
import json
import os

import ml_dtypes
import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    out = {}
    codes = np.arange(256, dtype=np.uint8)
    dec_t = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    dec_m = codes.view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    assert np.array_equal(np.nan_to_num(dec_t, nan=9e9), np.nan_to_num(dec_m, nan=9e9))
    out["e4m3fn_decode_bits"] = dec_t.view(np.uint32).tolist()      # fp32 bit patterns of all 256 codes

    # encode of every bf16 bit pattern (saturating, RN-even); NaN inputs -> 0x7F
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    x = (bits.astype(np.uint32) << 16).view(np.float32)
    nan = np.isnan(x)
    xc = np.clip(np.nan_to_num(x, nan=0.0), -448, 448)
    enc_t = torch.from_numpy(xc).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    enc_m = xc.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    assert np.array_equal(enc_t, enc_m)
    enc_t = enc_t.copy()
    enc_t[nan] = 0x7F
    np.save(os.path.join(HERE, "e4m3fn_encode_of_bf16.npy"), enc_t)

    # hand-picked fp32 encode cases: ties, subnormals, saturation
    cases = [0.0, -0.0, 1.0, 1.0625, 1.0626, 1.1875, 0.001953125, 0.0009765625, 0.00097656256, 0.0029296875,
             0.015625, 0.0146484375, 448.0, 464.0, 480.0, 1e9, -1e9, 240.0, 247.9, 248.0, -3.3, 17.0, 18.0, 19.0,
             float("inf"), float("-inf")]
    xs = np.array(cases, np.float32)
    e = torch.from_numpy(np.clip(xs, -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    out["encode_cases"] = {"x_bits": xs.view(np.uint32).tolist(), "code": e.tolist()}

    # bf16 rounding cases
    r = np.random.default_rng(7).standard_normal(4096).astype(np.float32) * np.float32(37.0)
    r[:6] = [1.00390625, 1.01171875, 3.0e38, -1.0e-40, 0.0, 65504.0]
    b = torch.from_numpy(r).bfloat16().view(torch.int16).numpy().view(np.uint16)
    out["bf16_cases"] = {"x_bits": r.view(np.uint32).tolist(), "bf16": b.tolist()}

    # tiny GEMMs with exact small-integer answers (the reference's commented
    # probes: one-hot / constant rows).  Codes: 0x38=1, 0x40=2, 0x30=0.5, 0xB8=-1
    M, N, K = 3, 6, 32
    A = np.full((M, K), 0x38, np.uint8)
    A[1, :] = 0
    A[1, 5] = 0x40
    A[2, ::2] = 0xB8
    B = np.zeros((N, K), np.uint8)
    for j in range(N):
        B[j, :] = [0x38, 0x40, 0x30, 0xB8, 0x38, 0x48][j]        # 1, 2, .5, -1, 1, 4
    B[4, 5] = 0x50                                              # 8
    Af = torch.from_numpy(A).view(torch.float8_e4m3fn).double()
    Bf = torch.from_numpy(B).view(torch.float8_e4m3fn).double()
    D = (Af @ Bf.T) * 0.5 * 0.25
    out["tiny_gemm"] = {"A": A.tolist(), "B": B.tolist(), "scale_a": 0.5, "scale_b": 0.25,
                        "D_bf16": D.float().bfloat16().view(torch.int16).numpy().view(np.uint16).tolist()}

    # block-128 quantisation of a seeded bf16 vector, computed with torch
    g = torch.Generator().manual_seed(11)
    xb = torch.randn(1024, generator=g).bfloat16()
    xb[128:256] = 0
    xb[300] = 1e4
    f = xb.float().reshape(-1, 128)
    amax = f.abs().amax(1, keepdim=True)
    s = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (f / s).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    out["blocks128"] = {"x_bf16": xb.view(torch.int16).numpy().view(np.uint16).tolist(),
                        "q": q.reshape(-1).tolist(), "scale_bits": s.reshape(-1).numpy().view(np.uint32).tolist()}

    with open(os.path.join(HERE, "known_answers.json"), "w") as fjson:
        json.dump(out, fjson)
    print("wrote", sorted(out))


if __name__ == "__main__":
    main()
