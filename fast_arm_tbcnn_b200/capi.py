"""ctypes binding of include/tbn_cuda.h.

Device memory comes from torch (``tensor.data_ptr()``); torch is plumbing only -- every
computation below runs in the library's own kernels.  There is no fallback: if the shared
library is missing ``load()`` raises, and every call checks the returned status.
"""
import ctypes as C
import os

from . import build as _build

EPI_ADD_RESIDUAL = 4
MODE_AUTO, MODE_TC_BF16X1, MODE_TC_BF16X2, MODE_TC_BF16X3, MODE_SIMT, MODE_TC_FP16X1 = 0, 1, 2, 3, 4, 5
EPI_RELU, EPI_BIAS_BEFORE_ALPHA = 1, 2
LAYOUT_KN, LAYOUT_NK = 0, 1
CONV_WEIGHTS_REFERENCE, CONV_WEIGHTS_TAP_MAJOR = 0, 1
ELT_GREATER, ELT_LESS, ELT_SUB = 0, 1, 2

_vp, _i64, _i32, _f32, _u32, _sz = C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_uint32, C.c_size_t

#: name -> (restype, argtypes); must list every symbol include/tbn_cuda.h declares.
SIGNATURES = {
    "tbn_cuda_init": (_i32, [_i32]),
    "tbn_cuda_last_error": (_i32, [C.c_char_p, _sz]),
    "tbn_cuda_malloc": (_i32, [C.POINTER(_vp), _sz]),
    "tbn_cuda_free": (_i32, [_vp]),
    "tbn_cuda_memset": (_i32, [_vp, _i32, _sz, _vp]),
    "tbn_cuda_h2d": (_i32, [_vp, _vp, _sz, _vp]),
    "tbn_cuda_d2h": (_i32, [_vp, _vp, _sz, _vp]),
    "tbn_cuda_d2d": (_i32, [_vp, _vp, _sz, _vp]),
    "tbn_cuda_sync": (_i32, [_vp]),
    "tbn_cuda_launch_count": (_i64, []),
    "tbn_cuda_set_wait_limit_ns": (_i32, [C.c_uint64]),
    "tbn_cuda_selftest_wait_timeout": (_i32, [_vp]),
    "tbn_cuda_profile_enable": (_i32, [_i32]),
    "tbn_gemm_plan": (_i32, [_i64, _i64, _i64, C.POINTER(_i32), C.POINTER(_i32), C.POINTER(_i32), C.POINTER(_i32)]),
    "tbn_gemm_plan_override": (_i32, [_i32, _i32, _i32, _i32]),
    "tbn_gemm_plan_bn": (_i32, [_i64, _i64, _i32]),
    "tbn_cuda_set_fused_split": (_i32, [_i32]),
    "tbn_cuda_profile_read": (_i32, [C.POINTER(C.c_double), C.POINTER(_i64), C.POINTER(C.c_double), C.POINTER(_i64)]),
    "tbn_dense_pack_bytes": (_sz, [_i64, _i64]),
    "tbn_dense_pack": (_i32, [_vp, _i64, _i64, _i64, _i32, _vp, _vp]),
    "tbn_gemm_f32": (_i32, [_vp, _i64, _i64, _i64, _vp, _i64, _f32, _vp, _vp, _i64, _u32, _vp, _sz, _vp]),
    "tbn_conv2d_f32": (_i32, [_vp, _i64, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp,
                              _vp, _u32, _i32, _vp, _sz, _vp]),
    "tbn_conv2d_fxb_chain": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32,
                                    _i32, _vp, _f32, _vp, _vp, _vp, _vp, _i32, _u32, _i32, _vp, _sz, _vp]),
    "tbn_conv2d_f32_chain": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32,
                                    _i32, _vp, _vp, _vp, _vp, _u32, _i32, _vp, _sz, _vp]),
    "tbn_conv2d_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32]),
    "tbn_permute_filters": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp]),
    "tbn_conv2d_fxb": (_i32, [_vp, _i64, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32,
                              _vp, _f32, _vp, _vp, _vp, _i32, _u32, _i32, _vp, _sz, _vp]),
    "tbn_conv2d_tbn": (_i32, [_vp, _i64, _i64, _i64, _i64, _f32, _f32, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32,
                              _i32, _vp, _f32, _vp, _vp, _u32, _i32, _vp, _sz, _vp]),
    "tbn_lenet_fused_fxb": (_i32, [_vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tbn_relu": (_i32, [_vp, _i64, _vp, _vp]),
    "tbn_add": (_i32, [_vp, _i64, _vp, _i64, _i64, _i32, _vp, _vp]),
    "tbn_pool2d": (_i32, [_i32, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "tbn_global_avgpool2d": (_i32, [_vp, _i64, _i64, _i64, _i64, _vp, _vp]),
    "tbn_global_maxpool2d": (_i32, [_vp, _i64, _i64, _i64, _i64, _vp, _vp]),
    "tbn_binary_elementwise": (_i32, [_i32, _vp, _i64, _vp, _i64, _vp, _vp]),
    "tbn_transpose2d": (_i32, [_vp, _i64, _i64, _vp, _vp]),
    "tbn_gather_cols_permute": (_i32, [_vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "tbn_ipc_export": (_i32, [_vp, _vp]),
    "tbn_ipc_open": (_i32, [_vp, C.POINTER(_vp)]),
    "tbn_ipc_close": (_i32, [_vp]),
    "tbn_packed_dims": (_i32, [_i64, _i64, C.POINTER(_i64), C.POINTER(_i64)]),
    "tbn_quantize_to_binary": (_i32, [_vp, _i64, _f32, _vp, _vp]),
    "tbn_quantize_to_ternary": (_i32, [_vp, _i64, _f32, _f32, _vp, _vp]),
    "tbn_channel_abs_mean": (_i32, [_vp, _i64, _i64, _vp, _vp]),
    "tbn_quant_pack_workspace_bytes": (_sz, [_i64, _i64, _i32]),
    "tbn_quant_pack_binary": (_i32, [_vp, _i64, _i64, _i64, _i32, _f32, _i32, _vp, _vp, _vp, _sz, _vp]),
    "tbn_quant_pack_binary_noalloc": (_i32, [_vp, _i64, _i64, _i64, _i32, _f32, _i32, _vp, _vp, _vp]),
    "tbn_quant_pack_ternary": (_i32, [_vp, _i64, _i64, _i64, _i32, _f32, _f32, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "tbn_gemm_workspace_bytes": (_sz, [_i64, _i64, _i32]),
    "tbn_gemm_fxb": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _f32, _vp, _vp, _i64, _i32, _u32, _vp, _sz, _vp]),
    "tbn_gemm_fxb_multi": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _f32, _vp, C.POINTER(_vp), _i32, _i64, _i32, _u32,
                                  _vp, _sz, _vp]),
    "tbn_gemm_fxb_host_workspace_bytes": (_sz, [_i64, _i64, _i64, _i32]),
    "tbn_gemm_fxb_host": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _f32, _vp, _vp, _i64, _i32, _u32, _vp, _sz, _vp]),
    "tbn_gemm_tbn": (_i32, [_vp, _i64, _i64, _i64, _f32, _f32, _vp, _i64, _vp, _f32, _vp, _vp, _i64, _u32, _vp, _sz, _vp]),
}


class TbnError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"tbn_cuda status {status}: {message}")
        self.status = status


_LIB = None


def load(path=None):
    """Loads lib/libtbn_cuda.so (building it first when the sources are newer and nvcc exists)."""
    global _LIB
    if _LIB is not None and path is None:
        return _LIB
    path = path or _build.LIB_PATH
    if not os.path.exists(path):
        try:
            _build.build()
        except Exception as exc:  # noqa: BLE001
            raise ImportError(f"{path} is missing and could not be built: {exc}") from exc
    handle = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)  # AttributeError if the library does not export it
        fn.restype, fn.argtypes = res, args
    _LIB = handle
    return handle


def last_error():
    buf = C.create_string_buffer(1024)
    load().tbn_cuda_last_error(buf, 1024)
    return buf.value.decode(errors="replace")


def check(status):
    if status != 0:
        raise TbnError(status, last_error())


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class _Lib:
    """Tensor-level convenience wrappers (torch CUDA tensors in, torch CUDA tensors out)."""

    def __init__(self):
        self._inited = set()

    @property
    def h(self):
        return load()

    def init(self, device=None):
        import torch
        if device is None:
            device = torch.cuda.current_device()
        if device not in self._inited:
            check(self.h.tbn_cuda_init(device))
            self._inited.add(device)
        return device

    def sync(self):
        check(self.h.tbn_cuda_sync(_stream()))

    def launch_count(self):
        return int(self.h.tbn_cuda_launch_count())

    def set_fused_split(self, value=1):
        """0: always run the separate activation-split kernel; 1 (default): split inside the GEMM when N <= 256;
        2: split inside the GEMM whenever A's alignment allows."""
        check(self.h.tbn_cuda_set_fused_split(int(value)))

    def gemm_plan(self, M, N, K):
        """The library's per-shape choice for TBN_MODE_AUTO -> dict(kernel, bn, group_m, fused_split)."""
        k, b, g, f = _i32(), _i32(), _i32(), _i32()
        check(self.h.tbn_gemm_plan(M, N, K, C.byref(k), C.byref(b), C.byref(g), C.byref(f)))
        return {"kernel": ("tcgen05", "cuda-core", "tcgen05-pair")[k.value], "bn": b.value, "group_m": g.value,
                "fused_split": bool(f.value)}

    def wave_model_bn(self, M, N, preferred):
        return int(self.h.tbn_gemm_plan_bn(M, N, preferred))

    def describe_choice(self, M, N, K):
        return self.gemm_plan(M, N, K)

    def gemm_plan_override(self, kernel=-1, bn=-1, group_m=-1, fused_split=-1):
        check(self.h.tbn_gemm_plan_override(int(kernel), int(bn), int(group_m), int(fused_split)))

    def profile_enable(self, on=True):
        check(self.h.tbn_cuda_profile_enable(int(on)))

    def profile_read(self):
        """-> dict(gemm_ms, gemm_launches, split_ms, split_launches) since the last read."""
        g, gn, s, sn = C.c_double(), _i64(), C.c_double(), _i64()
        check(self.h.tbn_cuda_profile_read(C.byref(g), C.byref(gn), C.byref(s), C.byref(sn)))
        return {"gemm_ms": g.value, "gemm_launches": gn.value, "split_ms": s.value, "split_launches": sn.value}

    def gather_cols_permute(self, slabs, out=None):
        """slabs [G, M, Nc] -> out [M, G*Nc]."""
        import torch
        self.init()
        G, M, Nc = slabs.shape
        if out is None:
            out = torch.empty((M, G * Nc), dtype=torch.float32, device=slabs.device)
        check(self.h.tbn_gather_cols_permute(_ptr(slabs), G, M, Nc, _ptr(out), out.stride(0), _stream()))
        return out

    @staticmethod
    def packed_dims(K, N):
        return (K + 127) // 128 * 128, (N + 7) // 8 * 8

    # ---- quantise / pack --------------------------------------------------------------
    def quantize_to_binary(self, w, thr=0.0):
        import torch
        self.init()
        w = w.contiguous()
        out = torch.empty(w.shape, dtype=torch.uint8, device=w.device)
        check(self.h.tbn_quantize_to_binary(_ptr(w), w.numel(), thr, _ptr(out), _stream()))
        return out

    def quantize_to_ternary(self, w, lo=-0.1, hi=0.1):
        import torch
        self.init()
        w = w.contiguous()
        out = torch.empty(w.shape, dtype=torch.int8, device=w.device)
        check(self.h.tbn_quantize_to_ternary(_ptr(w), w.numel(), lo, hi, _ptr(out), _stream()))
        return out

    def channel_abs_mean(self, w):
        """[channels, ...] -> [channels] mean |w| per channel, sequential fp32 (bit-equal to the reference)."""
        import torch
        self.init()
        w = w.contiguous()
        ch = w.shape[0]
        out = torch.empty(ch, dtype=torch.float32, device=w.device)
        check(self.h.tbn_channel_abs_mean(_ptr(w), ch, w.numel() // ch, _ptr(out), _stream()))
        return out

    def quant_pack_binary(self, w, layout=LAYOUT_KN, thr=0.0, ge=False, want_alpha=True):
        """-> (words int32-viewed-as-uint32 [N_pad, K_pad/32], alpha [N] or None)."""
        import torch
        self.init()
        assert w.dim() == 2 and w.dtype == torch.float32 and w.stride(1) == 1
        K, N = (w.shape if layout == LAYOUT_KN else (w.shape[1], w.shape[0]))
        Kp, Np = self.packed_dims(K, N)
        words = torch.empty((Np, Kp // 32), dtype=torch.int32, device=w.device)
        alpha = torch.empty(N, dtype=torch.float32, device=w.device) if want_alpha else None
        ws_bytes = self.h.tbn_quant_pack_workspace_bytes(K, N, 0) if want_alpha else 0
        ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=w.device)
        check(self.h.tbn_quant_pack_binary(_ptr(w), K, N, w.stride(0), layout, thr, int(ge), _ptr(words), _ptr(alpha),
                                           _ptr(ws), ws_bytes, _stream()))
        return words, alpha

    def quant_pack_binary_noalloc(self, w, words, alpha, layout=LAYOUT_KN, thr=0.0, ge=False):
        """Variant that allocates nothing: the caller passes the outputs (`words` int32
        [N_pad, K_pad/32], `alpha` float32 [N] or None); the scratch is built into the library."""
        self.init()
        K, N = (w.shape if layout == LAYOUT_KN else (w.shape[1], w.shape[0]))
        check(self.h.tbn_quant_pack_binary_noalloc(_ptr(w), K, N, w.stride(0), layout, thr, int(ge), _ptr(words),
                                                   _ptr(alpha), _stream()))

    def quant_pack_ternary(self, w, lo, hi, layout=LAYOUT_KN, want_alpha=True, want_codes=True):
        """-> (codes [(K*N+15)/16] or None, pos, neg [N_pad, K_pad/32], alpha [N] or None)."""
        import torch
        self.init()
        assert w.dim() == 2 and w.dtype == torch.float32 and w.stride(1) == 1
        K, N = (w.shape if layout == LAYOUT_KN else (w.shape[1], w.shape[0]))
        Kp, Np = self.packed_dims(K, N)
        pos = torch.empty((Np, Kp // 32), dtype=torch.int32, device=w.device)
        neg = torch.empty_like(pos)
        codes = torch.empty((K * N + 15) // 16, dtype=torch.int32, device=w.device) if want_codes else None
        alpha = torch.empty(N, dtype=torch.float32, device=w.device) if want_alpha else None
        ws_bytes = self.h.tbn_quant_pack_workspace_bytes(K, N, 1) if want_alpha else 0
        ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=w.device)
        check(self.h.tbn_quant_pack_ternary(_ptr(w), K, N, w.stride(0), layout, lo, hi, _ptr(codes), _ptr(pos), _ptr(neg),
                                            _ptr(alpha), _ptr(ws), ws_bytes, _stream()))
        return codes, pos, neg, alpha

    # ---- GEMM ---------------------------------------------------------------------------
    def gemm_workspace(self, M, K, mode, device):
        import torch
        nbytes = self.h.tbn_gemm_workspace_bytes(M, K, mode)
        return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device), nbytes

    def gemm_fxb(self, a, neg, N, pos=None, alpha=None, scale=1.0, bias=None, mode=MODE_AUTO, epilogue=0, out=None,
                 workspace=None):
        import torch
        self.init()
        assert a.dim() == 2 and a.dtype == torch.float32 and a.stride(1) == 1
        M, K = a.shape
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=a.device)
        if workspace is None:
            workspace, nbytes = self.gemm_workspace(M, K, mode, a.device)
        else:
            nbytes = workspace.numel() * workspace.element_size()
        check(self.h.tbn_gemm_fxb(_ptr(a), M, K, a.stride(0), _ptr(neg), _ptr(pos), N, _ptr(alpha), scale, _ptr(bias),
                                  _ptr(out), out.stride(0), mode, epilogue, _ptr(workspace), nbytes, _stream()))
        return out

    def gemm_fxb_multi(self, a, neg, N, dest_ptrs, ldc, pos=None, alpha=None, scale=1.0, bias=None,
                       mode=MODE_TC_BF16X2, epilogue=0, workspace=None):
        """Column-slab GEMM whose epilogue stores the slab to every address in `dest_ptrs` (ints: device
        pointers, local and peer-mapped, already offset to the slab's first column; row stride `ldc`)."""
        self.init()
        M, K = a.shape
        if workspace is None:
            workspace, nbytes = self.gemm_workspace(M, K, mode, a.device)
        else:
            nbytes = workspace.numel() * workspace.element_size()
        arr = (_vp * len(dest_ptrs))(*[int(p) for p in dest_ptrs])
        check(self.h.tbn_gemm_fxb_multi(_ptr(a), M, K, a.stride(0), _ptr(neg), _ptr(pos), N, _ptr(alpha), scale, _ptr(bias),
                                        arr, len(dest_ptrs), ldc, mode, epilogue, _ptr(workspace), nbytes, _stream()))

    def gemm_fxb_host(self, a_host, neg, N, out_host, pos=None, alpha=None, scale=1.0, bias=None, mode=MODE_TC_BF16X2,
                      epilogue=0, workspace=None, device=None):
        """Host tensors in and out (torch CPU tensors, ideally pinned); weights on the device.  Asynchronous:
        synchronise the current stream before reading `out_host`."""
        import torch
        self.init()
        M, K = a_host.shape
        nbytes = self.h.tbn_gemm_fxb_host_workspace_bytes(M, K, N, mode)
        if workspace is None:
            workspace = torch.empty(nbytes, dtype=torch.uint8, device=device or neg.device)
        check(self.h.tbn_gemm_fxb_host(_ptr(a_host), M, K, a_host.stride(0), _ptr(neg), _ptr(pos), N, _ptr(alpha), scale,
                                       _ptr(bias), _ptr(out_host), out_host.stride(0), mode, epilogue, _ptr(workspace),
                                       workspace.numel(), _stream()))
        return out_host

    def gemm_tbn(self, a, neg, N, lo=-0.1, hi=0.1, alpha=None, scale=1.0, bias=None, epilogue=0, out=None,
                 workspace=None):
        import torch
        self.init()
        assert a.dim() == 2 and a.dtype == torch.float32 and a.stride(1) == 1
        M, K = a.shape
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=a.device)
        if workspace is None:
            workspace, nbytes = self.gemm_workspace(M, K, MODE_TC_BF16X1, a.device)
        else:
            nbytes = workspace.numel() * workspace.element_size()
        check(self.h.tbn_gemm_tbn(_ptr(a), M, K, a.stride(0), lo, hi, _ptr(neg), N, _ptr(alpha), scale, _ptr(bias),
                                  _ptr(out), out.stride(0), epilogue, _ptr(workspace), nbytes, _stream()))
        return out


    # ---- convolution and glue ops -----------------------------------------------------------
    @staticmethod
    def conv_out_hw(H, W, kh, kw, p):
        sh, sw, ph, pw, dh, dw = p
        if sh <= 0 or sw <= 0:
            return 0, 0  # the library rejects the call; the output shape does not matter
        return (H + 2 * ph - dh * (kh - 1) - 1) // sh + 1, (W + 2 * pw - dw * (kw - 1) - 1) // sw + 1

    def conv_workspace(self, xshape, m_out, kh, kw, device, order=CONV_WEIGHTS_REFERENCE):
        import torch
        N, Cc, H, W = xshape
        nbytes = self.h.tbn_conv2d_workspace_bytes(N, Cc, H, W, m_out, kh, kw, order)
        return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device), nbytes

    def permute_filters(self, w):
        """[M, C, kh, kw] -> [M, kh*kw*C] in tap-major order (for CONV_WEIGHTS_TAP_MAJOR)."""
        import torch
        self.init()
        w = w.contiguous()
        M, Cc, kh, kw = w.shape
        out = torch.empty((M, kh * kw * Cc), dtype=torch.float32, device=w.device)
        check(self.h.tbn_permute_filters(_ptr(w), M, Cc, kh * kw, _ptr(out), _stream()))
        return out

    def conv2d_fxb(self, x, neg, wshape, p, pos=None, alpha=None, scale=1.0, bias=None, residual=None, mode=MODE_AUTO,
                   epilogue=0, out=None, workspace=None, order=CONV_WEIGHTS_REFERENCE):
        """x [N,C,H,W]; packed weights of shape wshape = (M_out, C, kh, kw); p = (sh, sw, ph, pw, dh, dw)."""
        import torch
        self.init()
        x = x.contiguous()
        N, Cc, H, W = x.shape
        M_out, _, kh, kw = wshape
        oh, ow = self.conv_out_hw(H, W, kh, kw, p)
        if out is None:
            out = torch.empty((N, M_out, max(oh, 0), max(ow, 0)), dtype=torch.float32, device=x.device)
        if workspace is None:
            workspace, nbytes = self.conv_workspace(x.shape, M_out, kh, kw, x.device, order)
        else:
            nbytes = workspace.numel()
        if residual is not None:
            epilogue |= EPI_ADD_RESIDUAL
        check(self.h.tbn_conv2d_fxb(_ptr(x), N, Cc, H, W, _ptr(neg), _ptr(pos), M_out, kh, kw, *[int(v) for v in p],
                                    _ptr(alpha), scale, _ptr(bias), _ptr(residual), _ptr(out), mode, epilogue, order,
                                    _ptr(workspace), nbytes, _stream()))
        return out

    def conv2d_tbn(self, x, neg, wshape, p, lo=-0.1, hi=0.1, alpha=None, scale=1.0, bias=None, epilogue=0, out=None,
                   workspace=None, order=CONV_WEIGHTS_REFERENCE):
        import torch
        self.init()
        x = x.contiguous()
        N, Cc, H, W = x.shape
        M_out, _, kh, kw = wshape
        oh, ow = self.conv_out_hw(H, W, kh, kw, p)
        if out is None:
            out = torch.empty((N, M_out, max(oh, 0), max(ow, 0)), dtype=torch.float32, device=x.device)
        if workspace is None:
            workspace, nbytes = self.conv_workspace(x.shape, M_out, kh, kw, x.device, order)
        else:
            nbytes = workspace.numel()
        check(self.h.tbn_conv2d_tbn(_ptr(x), N, Cc, H, W, lo, hi, _ptr(neg), M_out, kh, kw, *[int(v) for v in p],
                                    _ptr(alpha), scale, _ptr(bias), _ptr(out), epilogue, order, _ptr(workspace), nbytes,
                                    _stream()))
        return out

    # ---- float weights ----------------------------------------------------------------------------
    def dense_pack(self, w, layout=LAYOUT_KN):
        """fp32 weights [K,N] (KN) or [N,K] (NK) -> split bf16 buffer (uint8 tensor)."""
        import torch
        self.init()
        assert w.dim() == 2 and w.dtype == torch.float32 and w.stride(1) == 1
        K, N = (w.shape if layout == LAYOUT_KN else (w.shape[1], w.shape[0]))
        buf = torch.empty(self.h.tbn_dense_pack_bytes(K, N), dtype=torch.uint8, device=w.device)
        check(self.h.tbn_dense_pack(_ptr(w), K, N, w.stride(0), layout, _ptr(buf), _stream()))
        return buf

    def gemm_f32(self, a, packed_w, N, alpha=1.0, bias=None, epilogue=0, out=None, workspace=None):
        import torch
        self.init()
        M, K = a.shape
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=a.device)
        if workspace is None:
            workspace, nbytes = self.gemm_workspace(M, K, MODE_TC_BF16X2, a.device)
        else:
            nbytes = workspace.numel()
        check(self.h.tbn_gemm_f32(_ptr(a), M, K, a.stride(0), _ptr(packed_w), N, alpha, _ptr(bias), _ptr(out), out.stride(0),
                                  epilogue, _ptr(workspace), nbytes, _stream()))
        return out

    def conv2d_f32(self, x, packed_w, wshape, p, bias=None, residual=None, epilogue=0, out=None, workspace=None,
                   order=CONV_WEIGHTS_REFERENCE):
        import torch
        self.init()
        x = x.contiguous()
        N, Cc, H, W = x.shape
        M_out, _, kh, kw = wshape
        oh, ow = self.conv_out_hw(H, W, kh, kw, p)
        if out is None:
            out = torch.empty((N, M_out, max(oh, 0), max(ow, 0)), dtype=torch.float32, device=x.device)
        if workspace is None:
            workspace, nbytes = self.conv_workspace(x.shape, M_out, kh, kw, x.device, order)
        else:
            nbytes = workspace.numel()
        if residual is not None:
            epilogue |= EPI_ADD_RESIDUAL
        check(self.h.tbn_conv2d_f32(_ptr(x), N, Cc, H, W, _ptr(packed_w), M_out, kh, kw, *[int(v) for v in p], _ptr(bias),
                                    _ptr(residual), _ptr(out), epilogue, order, _ptr(workspace), nbytes, _stream()))
        return out

    def conv2d_chain(self, xshape, w, wshape, p, x=None, x_cl=None, want_y=True, want_y_cl=False, alpha=None, scale=1.0,
                     bias=None, residual=None, epilogue=0, workspace=None, mode=MODE_TC_BF16X2, device=None):
        """Convolution inside a layer sequence (tap-major filters).  `w` is {"words": ...} (packed sign filters) or
        {"split": ...} (float filters).  Input: the NCHW fp32 tensor `x` or its channels-last bf16 terms `x_cl`
        [2, N, H, W, C] as written by a previous call.  Returns (y or None, y_cl or None)."""
        import torch
        self.init()
        N, Cc, H, W = xshape
        M_out, _, kh, kw = wshape
        device = device or (x.device if x is not None else x_cl.device)
        oh, ow = self.conv_out_hw(H, W, kh, kw, p)
        y = torch.empty((N, M_out, oh, ow), dtype=torch.float32, device=device) if want_y else None
        y_cl = torch.empty((2, N, oh, ow, M_out), dtype=torch.bfloat16, device=device) if want_y_cl else None
        if workspace is None:
            workspace, nbytes = self.conv_workspace(xshape, M_out, kh, kw, device, CONV_WEIGHTS_TAP_MAJOR)
        else:
            nbytes = workspace.numel()
        if residual is not None:
            epilogue |= EPI_ADD_RESIDUAL
        if x is not None:
            x = x.contiguous()
        if "words" in w:
            check(self.h.tbn_conv2d_fxb_chain(_ptr(x), _ptr(x_cl), N, Cc, H, W, _ptr(w["words"]), None, M_out, kh, kw,
                                              *[int(v) for v in p], _ptr(alpha), scale, _ptr(bias), _ptr(residual), _ptr(y),
                                              _ptr(y_cl), mode, epilogue, CONV_WEIGHTS_TAP_MAJOR, _ptr(workspace), nbytes,
                                              _stream()))
        else:
            check(self.h.tbn_conv2d_f32_chain(_ptr(x), _ptr(x_cl), N, Cc, H, W, _ptr(w["split"]), M_out, kh, kw,
                                              *[int(v) for v in p], _ptr(bias), _ptr(residual), _ptr(y), _ptr(y_cl), epilogue,
                                              CONV_WEIGHTS_TAP_MAJOR, _ptr(workspace), nbytes, _stream()))
        return y, y_cl

    def lenet_fused(self, x, w1, w2, wf, classes, out=None):
        """x [batch, 1, 28, 28]; w1 / w2 / wf: dicts with "words", "alpha" and optional "bias" (packed as the Session
        packs them).  One launch for the whole LeNet-shaped network -> logits [batch, classes]."""
        import torch
        self.init()
        x = x.contiguous()
        batch = x.shape[0]
        if out is None:
            out = torch.empty((batch, classes), dtype=torch.float32, device=x.device)
        check(self.h.tbn_lenet_fused_fxb(_ptr(x), batch, 6, 16, classes, _ptr(w1["words"]), _ptr(w1.get("alpha")), _ptr(w1.get("bias")),
                                         _ptr(w2["words"]), _ptr(w2.get("alpha")), _ptr(w2.get("bias")), _ptr(wf["words"]),
                                         _ptr(wf.get("alpha")), _ptr(wf.get("bias")), _ptr(out), _stream()))
        return out

    def relu(self, x):
        import torch
        self.init()
        x = x.contiguous()
        out = torch.empty_like(x)
        check(self.h.tbn_relu(_ptr(x), x.numel(), _ptr(out), _stream()))
        return out

    def add(self, a, b, relu=False):
        import torch
        self.init()
        a, b = a.contiguous(), b.contiguous()
        out = torch.empty_like(a)
        inner = a.shape[2] * a.shape[3] if (a.dim() == 4 and a.numel() != b.numel()) else 1
        check(self.h.tbn_add(_ptr(a), a.numel(), _ptr(b), b.numel(), inner, int(relu), _ptr(out), _stream()))
        return out

    def pool2d(self, kind, x, p, ceil_mode=False, count_include_pad=False):
        """kind 0 max / 1 average; p = (kh, kw, sh, sw, ph, pw)."""
        import torch
        self.init()
        x = x.contiguous()
        N, Cc, H, W = x.shape
        kh, kw, sh, sw, ph, pw = [int(v) for v in p]
        if ceil_mode:
            oh, ow = (H + 2 * ph - kh + sh - 1) // sh + 1, (W + 2 * pw - kw + sw - 1) // sw + 1
        else:
            oh, ow = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        out = torch.empty((N, Cc, oh, ow), dtype=torch.float32, device=x.device)
        check(self.h.tbn_pool2d(kind, _ptr(x), N, Cc, H, W, kh, kw, sh, sw, ph, pw, int(ceil_mode), int(count_include_pad),
                                _ptr(out), _stream()))
        return out

    def global_avgpool2d(self, x):
        import torch
        self.init()
        x = x.contiguous()
        N, Cc, H, W = x.shape
        out = torch.empty((N, Cc, 1, 1), dtype=torch.float32, device=x.device)
        check(self.h.tbn_global_avgpool2d(_ptr(x), N, Cc, H, W, _ptr(out), _stream()))
        return out

    def global_maxpool2d(self, x):
        import torch
        self.init()
        x = x.contiguous()
        N, Cc, H, W = x.shape
        out = torch.empty((N, Cc, 1, 1), dtype=torch.float32, device=x.device)
        check(self.h.tbn_global_maxpool2d(_ptr(x), N, Cc, H, W, _ptr(out), _stream()))
        return out

    def binary_elementwise(self, op, x, rhs):
        """op: ELT_GREATER / ELT_LESS (float 0/1 result) or ELT_SUB; rhs is indexed modulo its length."""
        import torch
        self.init()
        x, rhs = x.contiguous(), rhs.contiguous()
        out = torch.empty_like(x)
        check(self.h.tbn_binary_elementwise(op, _ptr(x), x.numel(), _ptr(rhs), rhs.numel(), _ptr(out), _stream()))
        return out

    def transpose2d(self, x):
        import torch
        self.init()
        x = x.contiguous()
        out = torch.empty((x.shape[1], x.shape[0]), dtype=torch.float32, device=x.device)
        check(self.h.tbn_transpose2d(_ptr(x), x.shape[0], x.shape[1], _ptr(out), _stream()))
        return out


lib = _Lib()
