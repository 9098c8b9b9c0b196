"""Measures the GEMM kernel variants per shape class on the current GPU and writes the plan table.

    python -m fast_arm_tbcnn_b200.tune [--out-table csrc/gemm_plan_table.inc] [--out-report report.md] [--quick]

For one representative shape of every (M, N, K) class it times, with CUDA events and the override entry point
of the library (tbn_gemm_plan_override), the CUDA-core kernel and the tensor-core kernel with every column tile
(64 / 128 / 256), with and without the in-kernel activation split, and then the rasterisation groups for the
best of those.  The fastest variant becomes the class's line of the table that is compiled into the library
(rebuild after replacing csrc/gemm_plan_table.inc); the report lists every timing.  This is what replaces the
reference's auto_tune_gemm (tbn-runtime/src/operators/gemm.cpp:524-536), which tries CPU tile sizes.
"""
import argparse
import os
import sys

# One representative per class: the class's upper bound (the largest class: 16384), so that a choice is made for
# the heaviest shape it will serve.
M_REPS = [16, 128, 512, 2048, 8192, 16384]
N_REPS = [64, 128, 256, 1024, 4096, 16384]
K_REPS = [256, 1024, 4096, 16384]
M_CLASSES = ["<=16", "<=128", "<=512", "<=2048", "<=8192", ">8192"]
N_CLASSES = ["<=64", "<=128", "<=256", "<=1024", "<=4096", ">4096"]
K_CLASSES = ["<=256", "<=1024", "<=4096", ">4096"]
# Further shapes timed with the finished table against every explicit variant (they do not enter the table):
# the square ladder, the ternary projection and the GEMM views of the ResNet-18 layers at 64 images.
CHECK_SHAPES = [(n, n, n) for n in (128, 256, 512, 1024, 4096)] + [(4096, 11008, 4096)] + [
    (64 * 3136, 64, 576), (64 * 784, 128, 576), (64 * 784, 128, 1152), (64 * 196, 256, 1152), (64 * 196, 256, 2304),
    (64 * 49, 512, 2304), (64 * 49, 512, 4608), (64, 1000, 512)]


def main():
    ap = argparse.ArgumentParser()
    here = os.path.dirname(os.path.abspath(__file__))
    ap.add_argument("--out-table", default=os.path.join(here, "csrc", "gemm_plan_table.inc"))
    ap.add_argument("--out-report", default=None)
    ap.add_argument("--quick", action="store_true", help="skip the classes whose representative exceeds 2^40 multiply-adds")
    args = ap.parse_args()
    import torch
    from . import capi
    L = capi.lib
    L.init()
    dev = torch.device("cuda", torch.cuda.current_device())
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g = torch.Generator(device=dev).manual_seed(0)
    a_cache, w_cache = {}, {}

    def operands(M, N, K):
        if (M, K) not in a_cache:
            a_cache.clear()
            a_cache[(M, K)] = torch.randn((M, K), generator=g, device=dev)
        if (K, N) not in w_cache:
            w_cache.clear()
            w_cache[(K, N)] = L.quant_pack_binary(torch.randn((K, N), generator=g, device=dev))
        return a_cache[(M, K)], w_cache[(K, N)]

    def time_variant(M, N, K, kernel, bn=-1, group=-1, fused=-1):
        A, (words, alpha) = operands(M, N, K)
        out = torch.empty((M, N), device=dev)
        ws, _ = L.gemm_workspace(M, K, capi.MODE_TC_BF16X2, dev)
        work = 2.0 * M * N * K
        reps = 3 if work > 1e12 else (10 if work > 1e10 else 30)
        L.gemm_plan_override(kernel, bn, group, fused)
        try:
            mode = capi.MODE_AUTO
            for _ in range(2):
                L.gemm_fxb(A, words, N, alpha=alpha, mode=mode, out=out, workspace=ws)
            torch.cuda.synchronize()
            ev0.record()
            for _ in range(reps):
                L.gemm_fxb(A, words, N, alpha=alpha, mode=mode, out=out, workspace=ws)
            ev1.record()
            torch.cuda.synchronize()
            return ev0.elapsed_time(ev1) / reps
        finally:
            L.gemm_plan_override()

    def sweep(M, N, K):
        """-> (best variant, {variant: ms})."""
        timings = {}
        if M * N * K <= 2 ** 28 and M <= 65535 * 32:
            timings[("cuda-core", 0, 0, 0)] = time_variant(M, N, K, 1)
        bns = [b for b in (64, 128, 256) if b <= max(64, (N + 63) // 64 * 64)]
        for bn in bns:
            for fused in ((0, 1) if (N <= 1024 and K % 4 == 0) else (0,)):
                timings[("tcgen05", bn, 4, fused)] = time_variant(M, N, K, 0, bn, 4, fused)
        if M >= 256 and N >= 256:   # CTA pairs (cta_group::2): 256 x 256 tiles
            timings[("tcgen05-pair", 256, 4, 0)] = time_variant(M, N, K, 2, -1, 4, 0)
        best = min((k for k in timings if k[0] == "tcgen05"), key=lambda k: timings[k])
        if (M + 127) // 128 > 1 and (N + best[1] - 1) // best[1] > 1:
            for group in (1, 2, 8, 16):
                timings[("tcgen05", best[1], group, best[3])] = time_variant(M, N, K, 0, best[1], group, best[3])
        best = min(timings, key=lambda k: timings[k])
        # Run-to-run noise is a few per cent: the default rasterisation group (4) stays unless another one is
        # more than 2 % faster.
        dflt = (best[0], best[1], 4, best[3])
        if best[0] == "tcgen05" and best[2] != 4 and dflt in timings and timings[dflt] <= timings[best] * 1.02:
            best = dflt
        return best, timings

    lines, report = [], ["| class M | class N | class K | shape | chosen | ms | all variants (ms) |", "|---|---|---|---|---|---|---|"]
    for mi, M in enumerate(M_REPS):
        for ni, N in enumerate(N_REPS):
            for ki, K in enumerate(K_REPS):
                if args.quick and M * N * K > 2 ** 40:
                    continue
                best, timings = sweep(M, N, K)
                kernel = {"tcgen05": 0, "cuda-core": 1, "tcgen05-pair": 2}[best[0]]
                bn, group, fused = (best[1], best[2], best[3]) if kernel != 1 else (64, 4, 0)
                lines.append(f"{{{mi}, {ni}, {ki}, {kernel}, {bn}, {group}, {fused}}},")
                allv = "; ".join(f"{k[0]}" + (f" bn{k[1]} g{k[2]}" + (" fused" if k[3] else "") if k[0] != "cuda-core" else "") +
                                 f" {v:.4f}" for k, v in sorted(timings.items(), key=lambda kv: kv[1]))
                report.append(f"| {M_CLASSES[mi]} | {N_CLASSES[ni]} | {K_CLASSES[ki]} | {M}x{N}x{K} | {best[0]}"
                              + (f" bn{bn} g{group}" + (" fused" if fused else "") if kernel != 1 else "") +
                              f" | {timings[best]:.4f} | {allv} |")
                sys.stderr.write(report[-1] + "\n")
    header = ("// {class of M, class of N, class of K, kernel, bn, group_m, fused_split}; written by fast_arm_tbcnn_b200/tune.py.\n"
              "// Classes: M <=16 | <=128 | <=512 | <=2048 | <=8192 | larger;  N <=64 | <=128 | <=256 | <=1024 | <=4096 | larger;\n"
              "// K <=256 | <=1024 | <=4096 | larger.  A class without a line uses the built-in rule.\n")
    with open(args.out_table, "w") as f:
        f.write(header + "\n".join(lines) + "\n")
    # The table just measured, as the library would apply it (class entry + padding rule), against the best explicit
    # variant on shapes that are not class representatives.
    report += ["", "Shapes outside the table's representatives: the variant the new table selects against the best of all",
               "explicit variants (a ratio of 1.00 means the table's choice is the fastest measured).", "",
               "| shape MxNxK | table's variant | ms | best variant | ms | ratio |", "|---|---|---|---|---|---|"]
    table = {}
    for ln in lines:
        v = [int(x) for x in ln.strip("{},").split(",")]
        table[(v[0], v[1], v[2])] = v[3:]
    bounds_m, bounds_n, bounds_k = [16, 128, 512, 2048, 8192], [64, 128, 256, 1024, 4096], [256, 1024, 4096]

    def cls(v, b):
        for i, x in enumerate(b):
            if v <= x:
                return i
        return len(b)

    for (M, N, K) in CHECK_SHAPES:
        ent = table.get((cls(M, bounds_m), cls(N, bounds_n), cls(K, bounds_k)))
        if ent is None:
            continue
        best, timings = sweep(M, N, K)
        kernel, bn, group, fused = ent
        bn = L.wave_model_bn(M, N, bn)   # the adjustment the library applies to the class's tile
        mine = time_variant(M, N, K, kernel, bn if kernel == 0 else -1, group if kernel != 1 else -1, fused if kernel == 0 else -1)
        name = "cuda-core" if kernel == 1 else ("tcgen05-pair" if kernel == 2 else f"tcgen05 bn{bn} g{group}" + (" fused" if fused else ""))
        report.append(f"| {M}x{N}x{K} | {name} | {mine:.4f} | {best[0]} bn{best[1]} g{best[2]}{' fused' if best[3] else ''} | "
                      f"{timings[best]:.4f} | {mine / timings[best]:.2f} |")
        sys.stderr.write(report[-1] + "\n")
    if args.out_report:
        with open(args.out_report, "w") as f:
            f.write("\n".join(report) + "\n")
    print(args.out_table)


if __name__ == "__main__":
    main()
