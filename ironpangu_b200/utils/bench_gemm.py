"""Time the tcgen05 GEMM against torch.matmul (cuBLAS) on a few shapes; CUDA events, L2 flushed between runs.

    python -m ironpangu_b200.utils.bench_gemm [--shapes 4096x4096x4096,...]
"""
from __future__ import annotations

import argparse
import json

import torch


def time_fn(fn, flush, iters=10):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="4096x4096x4096,4096x2112x4096,4096x3072x4096,4096x4096x1536,8192x8192x8192,128x3072x4096")
    ap.add_argument("--two-sm", action="store_true", help="also time the CTA-pair kernel (shapes with M and N multiples of 256) and check it against the one-CTA kernel")
    ap.add_argument("--persistent-ar", action="store_true",
                    help="also time the persistent GEMM + all-reduce kernel at world 1 (its main loop and epilogue without any exchange)")
    args = ap.parse_args()
    from ironpangu_b200.ops.gemm import gemm, gemm_allreduce

    fab = None
    if args.persistent_ar:
        from ironpangu_b200.parallel.fabric import Fabric
        fab = Fabric(0, 1)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    out = []
    for s in args.shapes.split(","):
        M, N, K = map(int, s.split("x"))
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        t_ours = time_fn(lambda: gemm(a, b, out=c), flush)          # IFAB_GEMM_2SM=0 in the environment: the one-CTA kernel for every shape
        t_lib = time_fn(lambda: torch.matmul(a, b.T, out=c), flush)
        fl = 2.0 * M * N * K
        out.append({"shape": s, "ours_ms": round(t_ours, 4), "ours_tflops": round(fl / t_ours / 1e9, 1),
                    "cublas_ms": round(t_lib, 4), "cublas_tflops": round(fl / t_lib / 1e9, 1)})
        if args.two_sm and M % 256 == 0 and N % 256 == 0:
            from ironpangu_b200.ops.gemm import gemm_2sm

            st = torch.zeros(1, dtype=torch.int32, device="cuda")
            c2 = torch.empty_like(c)
            gemm(a, b, out=c)
            gemm_2sm(a, b, out=c2, status_ptr=st.data_ptr())
            torch.cuda.synchronize()
            out[-1].update({"two_sm_status": int(st[0]), "two_sm_equals_one_cta": bool(torch.equal(c, c2)),
                            "two_sm_max_abs_diff": float((c.float() - c2.float()).abs().max())})
            if int(st[0]) == 0:
                t2 = time_fn(lambda: gemm_2sm(a, b, out=c2), flush)
                out[-1].update({"two_sm_ms": round(t2, 4), "two_sm_tflops": round(fl / t2 / 1e9, 1)})
                c3 = torch.empty_like(c)
                gemm_2sm(a, b, out=c3, status_ptr=st.data_ptr(), persistent=True)
                torch.cuda.synchronize()
                out[-1].update({"two_sm_persistent_status": int(st[0]), "two_sm_persistent_equals_one_cta": bool(torch.equal(c, c3))})
                if int(st[0]) == 0:
                    t3 = time_fn(lambda: gemm_2sm(a, b, out=c3, persistent=True), flush)
                    out[-1].update({"two_sm_persistent_ms": round(t3, 4), "two_sm_persistent_tflops": round(fl / t3 / 1e9, 1)})
        if fab is not None:
            sym = fab.symmetric_empty((M, N))
            res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
            t_p = time_fn(lambda: gemm_allreduce(a, b, fab, sym, residual=res), flush)
            t_pn = time_fn(lambda: gemm_allreduce(a, b, fab, sym), flush)
            out[-1].update({"persistent_ar_world1_ms": round(t_p, 4), "persistent_ar_world1_tflops": round(fl / t_p / 1e9, 1),
                            "persistent_ar_world1_no_residual_ms": round(t_pn, 4)})
        print(json.dumps(out[-1]), flush=True)


if __name__ == "__main__":
    main()
