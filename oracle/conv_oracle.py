"""CPU restatement of the reference's convolution (forward and the two gradients) and average
pooling for C,D,H,W,N tensors.

TEST INFRASTRUCTURE ONLY (tests, smoke check, CPU-baseline legs of the bench).  Follows the numpy
fallbacks of the reference's CPU engine (ngraph/transformers/cpu/cpuengine.py:234-283 fprop_conv:
for every output position, dot of the clipped filter slice with the clipped input slice; :285-305
fprop_pool avg: mean of the clipped window) and ngraph/testing/conv_utils.py:66-102
(reference_conv).  Written tap-wise instead of position-wise: for every filter tap (r, s) one
tensordot over channels, which is the same sum in a different order.
The gradients follow ngraph/transformers/cpu/cpuengine.py:256-271 (bprop_conv: the same loop with
the filter flipped and transposed over the "backward" slices) and :395-418 (update_conv: for every
output position, outer product of the clipped input slice with the error column, accumulated).
Pinned against the reference CPU transformer's outputs in tests/golden/fixtures (conv_basic,
conv_stride2_*, conv_grads*, resnet*).
"""
import numpy as np


def conv_fprop(I, F, pad=(0, 0), stride=(1, 1), dtype=np.float32):
    """I: (C, H, W, N); F: (C, R, S, K) -> O: (K, P, Q, N).  dtype np.int64 gives the exact
    integer sums used for flex16 mantissas."""
    C, H, W, N = I.shape
    C2, R, S, K = F.shape
    assert C == C2
    ph, pw = pad
    sh, sw = stride
    P = (H + 2 * ph - R) // sh + 1
    Q = (W + 2 * pw - S) // sw + 1
    Ip = np.zeros((C, H + 2 * ph, W + 2 * pw, N), dtype=dtype)
    Ip[:, ph:ph + H, pw:pw + W, :] = I
    O = np.zeros((K, P, Q, N), dtype=dtype)
    Ft = F.astype(dtype)
    for r in range(R):
        for s in range(S):
            win = Ip[:, r:r + (P - 1) * sh + 1:sh, s:s + (Q - 1) * sw + 1:sw, :]
            O += np.tensordot(Ft[:, r, s, :].T, win, axes=([1], [0]))
    return O


def conv_bprop(E, F, in_hw, pad=(0, 0), stride=(1, 1), dtype=np.float32):
    """E: (K, P, Q, N); F: (C, R, S, K) -> gI: (C, H, W, N), the gradient of conv_fprop with
    respect to its input.  Every tap scatters F[:, r, s, :] . E onto the input positions it read."""
    K, P, Q, N = E.shape
    C, R, S, K2 = F.shape
    assert K == K2
    H, W = in_hw
    ph, pw = pad
    sh, sw = stride
    G = np.zeros((C, H + 2 * ph + R, W + 2 * pw + S, N), dtype=dtype)
    Ft = F.astype(dtype)
    Et = E.astype(dtype)
    for r in range(R):
        for s in range(S):
            G[:, r:r + (P - 1) * sh + 1:sh, s:s + (Q - 1) * sw + 1:sw, :] += np.tensordot(
                Ft[:, r, s, :], Et, axes=([1], [0]))
    return np.ascontiguousarray(G[:, ph:ph + H, pw:pw + W, :])


def conv_update(I, E, filter_hw, pad=(0, 0), stride=(1, 1), dtype=np.float32):
    """I: (C, H, W, N); E: (K, P, Q, N) -> U: (C, R, S, K), the gradient of conv_fprop with
    respect to its filters."""
    C, H, W, N = I.shape
    K, P, Q, N2 = E.shape
    assert N == N2
    R, S = filter_hw
    ph, pw = pad
    sh, sw = stride
    Ip = np.zeros((C, H + 2 * ph + R, W + 2 * pw + S, N), dtype=dtype)
    Ip[:, ph:ph + H, pw:pw + W, :] = I
    Et = E.astype(dtype)
    U = np.zeros((C, R, S, K), dtype=dtype)
    for r in range(R):
        for s in range(S):
            win = Ip[:, r:r + (P - 1) * sh + 1:sh, s:s + (Q - 1) * sw + 1:sw, :]
            U[:, r, s, :] = np.tensordot(win, Et, axes=([1, 2, 3], [1, 2, 3]))
    return U


def pool_avg_fprop(I, window, pad=(0, 0), stride=(1, 1)):
    """I: (C, H, W, N) -> (C, P, Q, N): mean over the part of each window inside the image."""
    C, H, W, N = I.shape
    R, S = window
    ph, pw = pad
    sh, sw = stride
    P = (H + 2 * ph - R) // sh + 1
    Q = (W + 2 * pw - S) // sw + 1
    O = np.zeros((C, P, Q, N), dtype=np.float32)
    for p in range(P):
        for q in range(Q):
            h0, h1 = max(p * sh - ph, 0), min(p * sh - ph + R, H)
            w0, w1 = max(q * sw - pw, 0), min(q * sw - pw + S, W)
            O[:, p, q, :] = I[:, h0:h1, w0:w1, :].reshape(C, -1, N).mean(axis=1)
    return O


def pool_max_fprop(I, window, pad=(0, 0), stride=(1, 1)):
    """I: (C, H, W, N) -> (C, P, Q, N): maximum over the part of each window inside the image
    (np.max of the same slices as the mean, ngraph/transformers/cpu/cpuengine.py:297-300)."""
    C, H, W, N = I.shape
    R, S = window
    ph, pw = pad
    sh, sw = stride
    P = (H + 2 * ph - R) // sh + 1
    Q = (W + 2 * pw - S) // sw + 1
    O = np.zeros((C, P, Q, N), dtype=I.dtype)
    for p in range(P):
        for q in range(Q):
            h0, h1 = max(p * sh - ph, 0), min(p * sh - ph + R, H)
            w0, w1 = max(q * sw - pw, 0), min(q * sw - pw + S, W)
            O[:, p, q, :] = I[:, h0:h1, w0:w1, :].reshape(C, -1, N).max(axis=1)
    return O


def pool_bprop(E, I, window, pad=(0, 0), stride=(1, 1), op="avg"):
    """E: (C, P, Q, N), I: (C, H, W, N) -> gradient of the pooling with respect to I, windows
    visited in (p, q) order as in ngraph/transformers/cpu/cpuengine.py:316-336.  avg: every
    in-image element of a window gets E * (1 / their number); max: the first maximum (np.argmax
    over the window in row-major order) gets E."""
    C, H, W, N = I.shape
    R, S = window
    ph, pw = pad
    sh, sw = stride
    P = (H + 2 * ph - R) // sh + 1
    Q = (W + 2 * pw - S) // sw + 1
    assert E.shape == (C, P, Q, N)
    G = np.zeros((C, H, W, N), dtype=np.float32)
    cols = np.arange(N)
    for p in range(P):
        for q in range(Q):
            h0, h1 = max(p * sh - ph, 0), min(p * sh - ph + R, H)
            w0, w1 = max(q * sw - pw, 0), min(q * sw - pw + S, W)
            for c in range(C):
                patch = G[c, h0:h1, w0:w1, :].reshape(-1, N).copy()
                if op == "max":
                    arg = np.argmax(I[c, h0:h1, w0:w1, :].reshape(-1, N), axis=0)
                    patch[arg, cols] += E[c, p, q, :]
                else:
                    patch += E[c, p, q, :] * np.float32(1.0 / patch.shape[0])
                G[c, h0:h1, w0:w1, :] = patch.reshape(h1 - h0, w1 - w0, N)
    return G


# ---- the same three contractions with the depth axes (D / T / M) and filter dilation ------------
def _out_extent(x, f, pad, stride, dil):
    return (x + 2 * pad - dil * (f - 1) - 1) // stride + 1


def conv3d_fprop(I, F, pad=(0, 0, 0), stride=(1, 1, 1), dil=(1, 1, 1), dtype=np.float32):
    """I: (C, D, H, W, N); F: (C, T, R, S, K) -> O: (K, M, P, Q, N); pad / stride / dil are
    (depth, height, width).  The reference's loop (ngraph/transformers/cpu/cpuengine.py:234-254)
    takes, for every output position, the dot of the clipped filter slice with the clipped input
    slice; here every filter tap contributes one tensordot over channels."""
    C, D, H, W, N = I.shape
    C2, T, R, S, K = F.shape
    assert C == C2
    (pd, ph, pw), (sd, sh, sw), (dd, dh, dw) = pad, stride, dil
    M, P, Q = _out_extent(D, T, pd, sd, dd), _out_extent(H, R, ph, sh, dh), _out_extent(W, S, pw, sw, dw)
    # padded so that every tap's strided window exists in full
    Ip = np.zeros((C, D + 2 * pd + sd, H + 2 * ph + sh, W + 2 * pw + sw, N), dtype=dtype)
    Ip[:, pd:pd + D, ph:ph + H, pw:pw + W, :] = I
    O = np.zeros((K, M, P, Q, N), dtype=dtype)
    Ft = F.astype(dtype)
    for t in range(T):
        for r in range(R):
            for s in range(S):
                win = Ip[:, t * dd:t * dd + (M - 1) * sd + 1:sd, r * dh:r * dh + (P - 1) * sh + 1:sh,
                         s * dw:s * dw + (Q - 1) * sw + 1:sw, :]
                O += np.tensordot(Ft[:, t, r, s, :].T, win, axes=([1], [0]))
    return O


def conv3d_bprop(E, F, in_dhw, pad=(0, 0, 0), stride=(1, 1, 1), dil=(1, 1, 1), dtype=np.float32):
    """E: (K, M, P, Q, N); F: (C, T, R, S, K) -> gI: (C, D, H, W, N): every tap scatters
    F[:, t, r, s, :] . E onto the input positions it read (the reference states it as the
    forward loop over flipped, transposed filters, cpuengine.py:256-271)."""
    K, M, P, Q, N = E.shape
    C, T, R, S, K2 = F.shape
    assert K == K2
    D, H, W = in_dhw
    (pd, ph, pw), (sd, sh, sw), (dd, dh, dw) = pad, stride, dil
    G = np.zeros((C, D + 2 * pd + T * dd + sd, H + 2 * ph + R * dh + sh, W + 2 * pw + S * dw + sw, N),
                 dtype=dtype)
    Ft, Et = F.astype(dtype), E.astype(dtype)
    for t in range(T):
        for r in range(R):
            for s in range(S):
                G[:, t * dd:t * dd + (M - 1) * sd + 1:sd, r * dh:r * dh + (P - 1) * sh + 1:sh,
                  s * dw:s * dw + (Q - 1) * sw + 1:sw, :] += np.tensordot(
                      Ft[:, t, r, s, :], Et, axes=([1], [0]))
    return np.ascontiguousarray(G[:, pd:pd + D, ph:ph + H, pw:pw + W, :])


def conv3d_update(I, E, filter_trs, pad=(0, 0, 0), stride=(1, 1, 1), dil=(1, 1, 1), dtype=np.float32):
    """I: (C, D, H, W, N); E: (K, M, P, Q, N) -> U: (C, T, R, S, K) (cpuengine.py:395-418)."""
    C, D, H, W, N = I.shape
    K, M, P, Q, N2 = E.shape
    assert N == N2
    T, R, S = filter_trs
    (pd, ph, pw), (sd, sh, sw), (dd, dh, dw) = pad, stride, dil
    Ip = np.zeros((C, D + 2 * pd + T * dd + sd, H + 2 * ph + R * dh + sh, W + 2 * pw + S * dw + sw, N),
                  dtype=dtype)
    Ip[:, pd:pd + D, ph:ph + H, pw:pw + W, :] = I
    Et = E.astype(dtype)
    U = np.zeros((C, T, R, S, K), dtype=dtype)
    for t in range(T):
        for r in range(R):
            for s in range(S):
                win = Ip[:, t * dd:t * dd + (M - 1) * sd + 1:sd, r * dh:r * dh + (P - 1) * sh + 1:sh,
                         s * dw:s * dw + (Q - 1) * sw + 1:sw, :]
                U[:, t, r, s, :] = np.tensordot(win, Et, axes=([1, 2, 3, 4], [1, 2, 3, 4]))
    return U
