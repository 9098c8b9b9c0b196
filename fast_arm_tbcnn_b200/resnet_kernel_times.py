"""Kernel times of one Session.run of the binary ResNet-18-style network (224 x 224), as they are inside the network.

    python -m fast_arm_tbcnn_b200.resnet_kernel_times [images per run = 512]

Runs the network three times under torch.profiler (CUDA activities) and prints, for the last run, every kernel with
its duration in launch order, then the sum.  A timing aid: unlike a profiler's launch list, which serialises the
kernels with cold caches, these are the durations of the back-to-back launches of an ordinary run.  Inputs are
torch.randn draws, weights the seeded recipe of graphs.resnet18.
"""
import sys


def main(argv):
    import torch
    from torch.profiler import ProfilerActivity, profile
    from . import graphs
    from .session import Session
    micro = int(argv[0]) if argv else 512
    sess = Session(graphs.resnet18(batch=micro, seed=2, image=224, classes=1000))
    sess.keep_intermediates = False
    sess.set_input("input", torch.randn((micro, 3, 224, 224), device="cuda"))
    for _ in range(2):
        sess.run()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(3):
            sess.run()
        torch.cuda.synchronize()
    kernels = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                     key=lambda e: e.time_range.start)
    per_run = len(kernels) // 3
    last = kernels[2 * per_run:]
    for e in last:
        print(f"{e.time_range.elapsed_us():9.1f} us  {e.name[:110]}")
    print(f"{per_run} kernels per run, {sum(e.time_range.elapsed_us() for e in last) / 1e3:.3f} ms in kernels")


if __name__ == "__main__":
    main(sys.argv[1:])
