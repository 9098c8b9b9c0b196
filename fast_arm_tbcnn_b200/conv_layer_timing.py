"""Times one float x binary 3x3 convolution layer (stride 1, pad 1, tap-major filters, two bf16 terms) on the current GPU.

    python -m fast_arm_tbcnn_b200.conv_layer_timing <batch> <C_in> <H = W> <C_out> [timed calls] [form]

`form` selects what the layer reads and writes: `nchw` (default: fp32 NCHW in and out, pre-pass included), or, as
inside a network (input already in channels-last bf16 terms, ReLU in the epilogue; needs C_in == C_out for the
residual): `cl` (writes the channels-last terms only), `y` (writes fp32 NCHW only), `y_cl` (both), `y_res` / `cl_res`
(one form plus a residual), `y_cl_res` (adds a residual and writes both forms -- the second convolution of a ResNet
block).

Prints the call time (CUDA events around back-to-back calls) and the kernel / pre-pass times from the library's own
per-kernel events (tbn_cuda_profile_enable).  TBN_CONV_ROWS=0 in the environment selects the patch-mode kernel
instead of the row-mode kernel, for comparisons.  Inputs are seeded torch.randn draws: this is a timing aid, parity
lives in tests/.
"""
import sys


def main(argv):
    import torch
    from . import capi
    L = capi.lib
    L.init()
    B, C, H, M = (int(v) for v in argv[:4])
    reps = int(argv[4]) if len(argv) > 4 else 5
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((B, C, H, H), generator=g, device="cuda")
    w = torch.randn((M, C, 3, 3), generator=g, device="cuda") * 0.05
    words, alpha = L.quant_pack_binary(L.permute_filters(w), capi.LAYOUT_NK)
    p = (1, 1, 1, 1, 1, 1)
    ws, _ = L.conv_workspace(x.shape, M, 3, 3, x.device, capi.CONV_WEIGHTS_TAP_MAJOR)
    y = torch.empty((B, M, H, H), device="cuda")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    form = argv[5] if len(argv) > 5 else "nchw"
    if form == "nchw":
        def call():
            L.conv2d_fxb(x, words, w.shape, p, alpha=alpha, workspace=ws, out=y, order=capi.CONV_WEIGHTS_TAP_MAJOR)
    else:
        wd = {"words": words}
        _, x_cl = L.conv2d_chain(tuple(x.shape), wd, tuple(w.shape), p, x=x, want_y=False, want_y_cl=True, alpha=alpha,
                                 epilogue=capi.EPI_RELU, workspace=ws)
        kw = {"cl": dict(want_y=False, want_y_cl=True), "y": dict(want_y=True, want_y_cl=False),
              "y_cl": dict(want_y=True, want_y_cl=True), "y_res": dict(want_y=True, want_y_cl=False, residual=x),
              "cl_res": dict(want_y=False, want_y_cl=True, residual=x),
              "y_cl_res": dict(want_y=True, want_y_cl=True, residual=x)}[form]

        def call():
            L.conv2d_chain(tuple(x.shape), wd, tuple(w.shape), p, x_cl=x_cl, alpha=alpha, epilogue=capi.EPI_RELU,
                           workspace=ws, **kw)

    L.profile_enable(True)
    for _ in range(2):
        call()
    torch.cuda.synchronize()
    L.profile_read()
    ev0.record()
    for _ in range(reps):
        call()
    ev1.record()
    torch.cuda.synchronize()
    pr = L.profile_read()
    L.profile_enable(False)
    flops = 2.0 * B * H * H * M * C * 9
    kernel = pr["gemm_ms"] / max(pr["gemm_launches"], 1)
    print(f"{C}x{H}x{H} -> {M}, batch {B}, {form}: call {ev0.elapsed_time(ev1) / reps:.4f} ms, kernel {kernel:.4f} ms, "
          f"pre-pass {pr['split_ms'] / max(pr['split_launches'], 1):.4f} ms, kernel {flops / kernel / 1e9:.1f} TFLOP/s")


if __name__ == "__main__":
    main(sys.argv[1:])
