"""Profiling target for Nsight Compute: a few launches of one operator on rotating weights.

    python -m lowbitlinear_b200.profile --operator gemv --shape 1x24576x4096 [--copies 4] [--launches 12]
    python -m lowbitlinear_b200.profile --operator gemm --shape 2048x24576x4096 --copies 1 --launches 3

Plays the role of the reference's ``benchmarks/profile_w4a16.py``: inputs are prepared and the
result is checked against an FP32 evaluation first, then the operator is launched ``--launches``
times, cycling through ``--copies`` distinct copies of the weights (so that a decode GEMV reads
HBM rather than the L2).  It reports no latency: timing under a profiler means nothing.  Keep
the case small (one kernel, a few launches, a few hundred MB) when capturing with
``ncu --set full --clock-control none -k regex:w4a16 -s <skip> -c <count>``.
"""
import argparse

import torch

from . import QuantizedLinear
from ._extension import load_cuda_extension


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--operator", choices=("gemv", "gemm"), required=True)
    parser.add_argument("--shape", required=True, help="MxNxK")
    parser.add_argument("--copies", type=int, default=4)
    parser.add_argument("--launches", type=int, default=12)
    parser.add_argument("--seed", type=int, default=42)
    args = parser.parse_args(argv)
    m, n, k = (int(v) for v in args.shape.lower().split("x"))
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA GPU")
    load_cuda_extension(required=True)
    torch.backends.cuda.matmul.allow_tf32 = False
    device = torch.device("cuda")
    g = torch.Generator(device=device).manual_seed(args.seed)
    x = torch.randn(m, k, device=device, generator=g).half()
    base = QuantizedLinear.from_float((torch.randn(n, k, device=device, generator=g) * 0.02).half())
    copies = [(base.packed_weight.clone(), base.scales.clone(), base.zeros.clone())
              for _ in range(max(1, args.copies))]

    def run(w):
        if args.operator == "gemv":
            return torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(x, *w, 64)
        return torch.ops.lowbitlinear_cute_w4a16.gemm(x, *w)

    shifts = torch.arange(8, device=device) * 4
    q = ((base.packed_weight.to(torch.int64)[..., None] >> shifts) & 15).reshape(n, -1)[:, :k]
    groups = torch.arange(k, device=device) // 64
    weight = (q.float() - base.zeros[:, groups].float()) * base.scales[:, groups]
    expected = (x.float() @ weight.T).half()
    actual = run(copies[0])
    rel = ((actual.float() - expected.float()).norm() / expected.float().norm()).item()
    assert rel <= 1e-3, f"relative L2 error {rel:.3e}"
    del q, weight
    for i in range(args.launches):
        out = run(copies[i % len(copies)])
    torch.cuda.synchronize()
    print(f"PASS {args.operator} shape={m}x{n}x{k} copies={len(copies)} launches={args.launches} "
          f"rel_l2={rel:.3e} checksum={float(out.float().abs().sum()):.4f}; no latency is reported here")


if __name__ == "__main__":
    main()
