"""Helpers shared by the parity tests."""
import numpy as np


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def pack_plane(mask_kn):
    """Boolean [K,N] -> uint32 words [ceil8(N), ceil128(K)/32] in the reference's binary-plane
    layout (word[n*(K_pad/32)+k/32], bit k%32), zero padded.  Independent numpy statement used
    to cross-check both the oracle and the CUDA packers."""
    K, N = mask_kn.shape
    Kp, Np = (K + 127) // 128 * 128, (N + 7) // 8 * 8
    full = np.zeros((Np, Kp), dtype=np.uint8)
    full[:N, :K] = mask_kn.T
    return np.packbits(full, axis=1, bitorder="little").view("<u4").reshape(Np, Kp // 32)


def special_weights(rng, K, N):
    """N(0,1) weights salted with the values whose classification is easy to get wrong."""
    w = rng.standard_normal((K, N), dtype=np.float32)
    specials = np.array([0.0, -0.0, np.nan, np.inf, -np.inf, 1e-45, -1e-45, 1e-39, 0.1, -0.1,
                         np.float32(0.1) + np.float32(1e-8), 0.25], dtype=np.float32)
    flat = w.reshape(-1)
    idx = rng.choice(flat.size, size=min(flat.size, 4 * specials.size), replace=False)
    flat[idx] = np.resize(specials, idx.size)
    return w


def u32(t):
    """torch int32 tensor (device) -> numpy uint32."""
    return t.cpu().numpy().view(np.uint32)
