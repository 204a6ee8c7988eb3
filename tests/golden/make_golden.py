"""Generates the golden fixtures in this directory by running the REFERENCE implementation.

Run once, in a container that has the reference checked out (it is not needed afterwards and
does not exist on the GPU machines):

    python tests/golden/make_golden.py --reference <checkout of NanjinLin/LowBitLinear>

The reference package (NanjinLin/LowBitLinear, ``lowbitlinear/``) is imported from that path
and nothing of it is copied: its ``quantize_int4`` / ``pack_int4`` / ``linear_int4_reference``
produce the tensors stored here, on CPU, from seeded inputs.

Files written:
  small_cases.npz   inputs and outputs of small layers (config "tiny" N=128 K=256 M=1 seed 0,
                    ragged K / N / group sizes, special value kinds), plus the GEMM-policy
                    output (weights rounded to FP16) computed with the reference's own
                    unpack/dequantise functions.
  full_size.json    for full Qwen3-8B-shaped linears: SHA-256 of packed words, scales and zero
                    points, and the first 64 outputs at M=1, so that the quantiser and the
                    oracle are pinned at benchmark size without storing 50 MB tensors.

Inputs come from ``torch.Generator('cpu').manual_seed(seed)``:  W = (randn(N, K) * std).half()
then x = randn(M, K).half() -- the recipe the benchmark and the tests share.
"""
import argparse
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

SMALL_CASES = [
    # name, M, N, K, group_size, weight std, seed
    ("tiny", 1, 128, 256, 64, 1.0, 0),
    ("ragged_k65", 16, 5, 65, 64, 1.0, 1),
    ("ragged_k70_g32", 5, 9, 70, 32, 1.0, 2),
    ("ragged_k129_g63", 9, 17, 129, 63, 1.0, 3),
    ("one", 1, 1, 1, 1, 1.0, 4),
    ("n130_k192", 3, 130, 192, 64, 0.02, 5),
    ("n129_k256", 1, 129, 256, 64, 0.02, 6),
    ("k512", 4, 48, 512, 64, 0.02, 7),
]
VALUE_KINDS = ["zero", "positive", "negative", "constant"]
FULL_SIZE = [
    # name, N, K, seed  (std 0.02, M = 1)
    ("o_proj", 4096, 4096, 1),
    ("down_proj", 4096, 12288, 3),
]


def seeded_inputs(m, n, k, std, seed):
    g = torch.Generator("cpu").manual_seed(seed)
    weight = (torch.randn(n, k, generator=g) * std).half()
    x = torch.randn(m, k, generator=g).half()
    return weight, x


def sha(t):
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="path of the reference checkout")
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    import lowbitlinear  # the reference package
    from lowbitlinear.linear import linear_int4_reference
    from lowbitlinear.quantization import dequantize_int4, pack_int4, quantize_int4, unpack_int4

    assert Path(lowbitlinear.__file__).resolve().is_relative_to(Path(args.reference).resolve())
    torch.backends.cuda.matmul.allow_tf32 = False

    arrays = {}

    def record(name, weight, x, group_size):
        q, scales, zeros = quantize_int4(weight, group_size)
        packed = pack_int4(q)
        y = linear_int4_reference(x, packed, scales, zeros, group_size)
        w_fp16 = dequantize_int4(unpack_int4(packed, original_k=weight.shape[1]), scales, zeros,
                                 group_size).half().float()
        y_mma = (x.float() @ w_fp16.T).half()
        arrays[f"{name}/weight"] = weight.numpy()
        arrays[f"{name}/x"] = x.numpy()
        arrays[f"{name}/group_size"] = np.int64(group_size)
        arrays[f"{name}/q"] = q.numpy()
        arrays[f"{name}/scales"] = scales.numpy()
        arrays[f"{name}/zeros"] = zeros.numpy()
        arrays[f"{name}/packed"] = packed.numpy()
        arrays[f"{name}/y"] = y.numpy()
        arrays[f"{name}/y_mma"] = y_mma.numpy()

    for name, m, n, k, gs, std, seed in SMALL_CASES:
        weight, x = seeded_inputs(m, n, k, std, seed)
        record(name, weight, x, gs)
    for i, kind in enumerate(VALUE_KINDS):
        weight, x = seeded_inputs(2, 3, 129, 1.0, 100 + i)
        weight = weight.float()
        if kind == "zero":
            weight.zero_()
        elif kind == "positive":
            weight.abs_()
        elif kind == "negative":
            weight = -weight.abs()
        elif kind == "constant":
            weight.fill_(2.5)
        record(f"kind_{kind}", weight, x, 63)
    np.savez_compressed(HERE / "small_cases.npz", **arrays)

    full = {}
    for name, n, k, seed in FULL_SIZE:
        weight, x = seeded_inputs(1, n, k, 0.02, seed)
        q, scales, zeros = quantize_int4(weight, 64)
        packed = pack_int4(q)
        y = linear_int4_reference(x, packed, scales, zeros, 64)
        full[name] = {
            "n": n, "k": k, "seed": seed, "std": 0.02, "m": 1,
            "weight_sha256": sha(weight), "x_sha256": sha(x),
            "packed_sha256": sha(packed), "scales_sha256": sha(scales),
            "zeros_sha256": sha(zeros),
            "y_first64_fp16_bits": y[0, :64].view(torch.int16).tolist(),
            "y_sha256": sha(y),
        }
    (HERE / "full_size.json").write_text(json.dumps(full, indent=1) + "\n")
    print("wrote", HERE / "small_cases.npz", (HERE / "small_cases.npz").stat().st_size, "bytes")
    print("wrote", HERE / "full_size.json")


if __name__ == "__main__":
    main()
