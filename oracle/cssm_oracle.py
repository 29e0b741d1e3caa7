"""CPU restatement (NumPy) of the CSSM spectral-SSM block forward pass.

TEST INFRASTRUCTURE ONLY.  Nothing that ships (the `cssm_b200` package) may import
this file; it is the checker for the CUDA path (tests, the smoke check and the
`cpu_baseline` / reference leg of the benchmark).

PINNED to the reference's own code: tests/golden/make_reference_golden.py imports the
reference's unmodified src/models/*.py on NumPy stand-ins for jax / flax.linen (oracle/_shim)
and stores what they compute in double precision; tests/test_reference_pin.py requires every
function here to reproduce those outputs to 1e-9 (all RoPE modes, gate types and activations,
kernel larger than the plane, ragged planes, the BASELINE block shapes, the GDN static-image
path, the scalar-scan blocks).  Further checks that need no reference checkout:
  * NumPy's FFT has the same conventions as `jnp.fft.rfft2/irfft2` (unnormalised
    forward, 1/(H*W) inverse, C2R ignoring the imaginary part of the DC / Nyquist
    columns);
  * a second, literal tier (`scan='goom'`) re-creates the reference's log-space
    (GOOM) scan arithmetic step by step in complex64, and the tests check it against
    the closed-form recurrence used by the first tier;
  * the reference's scan-operator tests (random |A|<1, U ~ N(0, .5^2), shapes from
    tests/test_complex32.py:81-93) and its sequential ground truth
    (benchmarks/bench_scan_modes.py:194-203) are re-expressed in tests/.

Reference lines followed (paths inside drewlinsley/CSSM):
  src/models/cssm.py:29-46      _stable_spectral_magnitude
  src/models/cssm.py:49-52      _rms_norm
  src/models/cssm.py:94-262     apply_rope
  src/models/cssm.py:353-383    apply_temporal_rope_to_context
  src/models/cssm.py:476-585    GatedCSSM._forward_depthwise
  src/models/cssm.py:4685-5141  GatedDeltaNetCSSM.__call__ (general path)
  src/models/goom.py:144-196    to_goom / from_goom (1e-7 magnitude floor)
  src/models/operations.py:17-61, 314-390  log_add_exp / log_sum_exp / block LMME
  src/models/math.py:24-54, 384-411        scan combine operators
Flax conventions honoured: Dense is x @ kernel + bias with kernel (in, out); Conv is
cross-correlation with HWIO kernels, 'SAME' pads (k-1)//2 low and k//2 high.
"""
from __future__ import annotations

import numpy as np

GOOM_EPS = 1e-7


# --------------------------------------------------------------------------- basics
def silu(x):
    return x * sigmoid(x)


def sigmoid(x):
    z = np.exp(-np.abs(x))                      # no overflow for large |x|
    return np.where(np.asarray(x) >= 0, 1.0 / (1.0 + z), z / (1.0 + z))


def softplus(x):
    return np.logaddexp(x, 0.0)


def dense(x, p):
    """flax.linen.Dense: x @ kernel + bias (kernel is (in, out))."""
    y = x @ p["kernel"].astype(x.dtype)
    if "bias" in p:
        y = y + p["bias"].astype(x.dtype)
    return y


def dwconv2d_same(x, p):
    """Depthwise cross-correlation, zero 'SAME' padding.  x (N,H,W,C); kernel (k,k,1,C).
    Follows nn.Conv(C, (k,k), feature_group_count=C, padding='SAME') at cssm.py:489-491."""
    k = p["kernel"].shape[0]
    lo, hi = (k - 1) // 2, k // 2
    N, H, W, C = x.shape
    xp = np.pad(x, ((0, 0), (lo, hi), (lo, hi), (0, 0)))
    w = p["kernel"].astype(x.dtype)
    out = np.zeros_like(x)
    for i in range(k):
        for j in range(k):
            out += xp[:, i:i + H, j:j + W, :] * w[i, j, 0, :]
    return out + p["bias"].astype(x.dtype)


def causal_tconv(x, p):
    """Causal depthwise 1-D conv over T.  x (B,T,H,W,C); kernel (k,1,C) (cssm.py:494-500).
    out[t] = b + sum_j w[j] * x[t-(k-1)+j], frames before t=0 are zero (padding happens
    after any earlier layer's bias, so a padded frame is exactly zero)."""
    k = p["kernel"].shape[0]
    B, T = x.shape[:2]
    xp = np.pad(x, ((0, 0), (k - 1, 0), (0, 0), (0, 0), (0, 0)))
    w = p["kernel"].astype(x.dtype)
    out = np.zeros_like(x)
    for j in range(k):
        out += xp[:, j:j + T] * w[j, 0, :]
    return out + p["bias"].astype(x.dtype)


# ----------------------------------------------------------------------------- RoPE
def rope_axis_freqs(C, mode, base=10000.0):
    """Per channel-pair angular frequencies (f_t, f_h, f_w), each (C/2,), such that the
    rotation angle of pair i at (t,h,w) is t*f_t[i] + h*f_h[i] + w*f_w[i].
    Restates the four branches of apply_rope (cssm.py:118-244) including the
    right-padding-with-zeros of the shorter h/w frequency lists."""
    n = C // 2
    inv = 1.0 / (base ** (np.arange(0, C, 2, dtype=np.float64) / C))
    ft = np.zeros(n); fh = np.zeros(n); fw = np.zeros(n)
    if mode == "none":
        pass
    elif mode == "temporal":
        ft[:] = inv
    elif mode == "spatial_only":
        a, b = inv[0::2], inv[1::2]
        fh[:len(a)] = a
        fw[:len(b)] = b
    elif mode == "mrope":
        nt = n // 3
        nh = n // 3
        th_t, th_h, th_w = inv[:nt], inv[nt:nt + nh], inv[nt + nh:]
        # interleave [t0,h0,w0,t1,h1,w1,...] then the remaining w frequencies
        for i in range(nt):
            ft[3 * i] = th_t[i]
            fh[3 * i + 1] = th_h[i]
            fw[3 * i + 2] = th_w[i]
        rest = th_w[nt:]
        fw[3 * nt:3 * nt + len(rest)] = rest
    elif mode == "spatiotemporal":
        nt = n // 3
        a, b = inv[nt::2], inv[nt + 1::2]
        ft[:nt] = inv[:nt]
        fh[:len(a)] = a
        fw[:len(b)] = b
    else:
        raise ValueError(f"unknown rope mode {mode!r}")
    return ft, fh, fw


def apply_rope(x, mode="spatiotemporal", base=10000.0):
    """cssm.py:94-262.  x (B,T,H,W,C)."""
    if mode == "none":
        return x
    B, T, H, W, C = x.shape
    ft, fh, fw = rope_axis_freqs(C, mode, base)
    th = (np.arange(T)[:, None, None, None] * ft
          + np.arange(H)[None, :, None, None] * fh
          + np.arange(W)[None, None, :, None] * fw)          # (T,H,W,C/2)
    c, s = np.cos(th).astype(x.dtype), np.sin(th).astype(x.dtype)
    xe, xo = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = xe * c - xo * s
    out[..., 1::2] = xe * s + xo * c
    return out


def temporal_ctx_code(T, C, base=10000.0):
    """cssm.py:353-383: interleaved (sin, cos) of t * inv_freq, shape (T, C)."""
    inv = 1.0 / (base ** (np.arange(0, C, 2, dtype=np.float64) / C))
    th = np.arange(T)[:, None] * inv[None, :]
    return np.stack([np.sin(th), np.cos(th)], axis=-1).reshape(T, C)


# ------------------------------------------------------------------ spectral kernel
def spectral_kernel(k, H, W, rho=0.999, squash=True):
    """Centre-pad (or centre-crop) a (C,ks,ks) kernel to (H,W), rfft2, squash the
    magnitude to < rho.  cssm.py:505-529 and :4713-4734, :29-46."""
    ks = k.shape[-1]
    if ks > H or ks > W:
        sh, sw = (ks - H) // 2, (ks - W) // 2
        kp = k[:, sh:sh + H, sw:sw + W]
    else:
        ph, pw = max(0, (H - ks) // 2), max(0, (W - ks) // 2)
        kp = np.pad(k, ((0, 0), (ph, max(0, H - ks - ph)), (pw, max(0, W - ks - pw))))
    K = np.fft.rfft2(kp.astype(np.float64), axes=(1, 2))
    if squash:
        K = K * rho / (1.0 + np.abs(K))
    return K


def goom_floor(z):
    """to_goom's magnitude floor (goom.py:161-173): |z| < 1e-7 -> 1e-7 + 0j."""
    z = np.asarray(z)
    zc = z.astype(np.complex128 if z.dtype in (np.float64, np.complex128) else np.complex64)
    return np.where(np.abs(zc) < GOOM_EPS, GOOM_EPS + 0j, zc)


# --------------------------------------------------- literal GOOM (log-space) scans
def _to_goom(z):
    z = np.asarray(z, dtype=np.complex64)
    z = np.where(np.abs(z) < np.float32(GOOM_EPS), np.complex64(GOOM_EPS), z)
    out = np.log(z).astype(np.complex64)
    floor = np.float32(np.log(np.finfo(np.float32).smallest_normal) * 2)
    return np.where(out.real < floor, floor + 1j * out.imag, out).astype(np.complex64)


def _from_goom(l):
    return np.exp(np.asarray(l, dtype=np.complex64)).astype(np.complex64)


def _log_add_exp(a, b):
    """operations.py:17-41."""
    c = np.maximum(a.real, b.real).astype(np.float32)
    x = _from_goom(a - c) + _from_goom(b - c)
    return (_to_goom(x) + c).astype(np.complex64)


def _log_sum_exp(l, axis):
    """operations.py:44-61."""
    c = np.max(l.real, axis=axis, keepdims=True).astype(np.float32)
    x = _from_goom(l - c).sum(axis=axis)
    return (_to_goom(x) + np.squeeze(c, axis=axis)).astype(np.complex64)


def goom_scalar_scan(A, U):
    """h_t = A_t h_{t-1} + U_t over axis 1, evaluated with the reference's log-space
    combine operator (math.py:24-54) applied left to right in complex64.  (Any
    bracketing of an associative operator gives the same value up to rounding;
    jax.lax.associative_scan uses a tree, this uses a chain.)"""
    Al, Ul = _to_goom(A), _to_goom(U)
    T = A.shape[1]
    out = [Ul[:, 0]]
    for t in range(1, T):
        out.append(_log_add_exp(Al[:, t] + out[-1], Ul[:, t]))
    return _from_goom(np.stack(out, axis=1))


def goom_matrix_scan(M, U):
    """u_t = M_t u_{t-1} + U_t with (.., d, d) matrices in log space
    (math.py:384-411, operations.py:355-390)."""
    Ml, Ul = _to_goom(M), _to_goom(U)
    T = M.shape[1]
    out = [Ul[:, 0]]
    for t in range(1, T):
        mv = _log_sum_exp(Ml[:, t] + out[-1][..., None, :], axis=-1)
        out.append(_log_add_exp(mv, Ul[:, t]))
    return _from_goom(np.stack(out, axis=1))


# ---------------------------------------------------------------------- gated block
def gate_activation(x, kind):
    """GatedCSSM._compute_gate, cssm.py:432-441."""
    if kind == "sigmoid":
        return sigmoid(x) * 2.0
    if kind == "exp":
        return np.exp(np.clip(x, -4, 2))
    return softplus(x)


def gated_forward(params, x, *, kernel_size, rope_mode="none", rope_base=10000.0,
                  spectral_rho=0.999, gate_activation_kind="softplus",
                  short_conv_size=4, short_conv_spatial_size=3, gate_type="dense",
                  dtype=np.float64, scan="direct", return_intermediates=False):
    """GatedCSSM.__call__ -> _forward_depthwise (cssm.py:443-474, 476-585).
    x (B,T,H,W,C) -> (B,T,H,W,C).

    scan='direct': h_t = A_t h_{t-1} + U_t as a plain complex FMA in `dtype`, with the
    GOOM magnitude floor applied to K_hat and to B*X_hat exactly where to_goom is
    called (cssm.py:559-563).  scan='goom': literal complex64 log-space arithmetic."""
    cdt = np.complex128 if dtype == np.float64 else np.complex64
    x = np.asarray(x, dtype=dtype)
    B, T, H, W, C = x.shape
    Wf = W // 2 + 1
    x = apply_rope(x, rope_mode, rope_base)
    xz = dense(x, params["in_proj"])
    x_main, z = xz[..., :C], xz[..., C:]
    if short_conv_spatial_size > 0:
        x_main = dwconv2d_same(x_main.reshape(B * T, H, W, C),
                               params["short_conv_spatial"]).reshape(B, T, H, W, C)
    if short_conv_size > 0:
        x_main = causal_tconv(x_main, params["short_conv_temporal"])
    x_main = silu(x_main)

    K_hat = spectral_kernel(params["kernel"], H, W, spectral_rho).astype(cdt)   # (C,H,Wf)
    U_hat = np.fft.rfft2(x_main.transpose(0, 1, 4, 2, 3), axes=(3, 4)).astype(cdt)
    ctx = x_main.mean(axis=(2, 3))                                              # (B,T,C)

    def make_gate(name):
        if gate_type == "factored":
            gh = dense(ctx, params[f"{name}_h"])
            gw = dense(ctx, params[f"{name}_w"])
            return (gh[..., :, None] * gw[..., None, :]).reshape(B, T, 1, H, Wf)
        return dense(ctx, params[name]).reshape(B, T, 1, H, Wf)

    delta = gate_activation(make_gate("delta_proj"), gate_activation_kind)
    Bg = make_gate("B_proj")
    Cg = make_gate("C_proj")

    if scan == "goom":
        K_log = _to_goom(K_hat)
        K_log = np.broadcast_to(K_log[None, None], U_hat.shape)
        U_log = _to_goom(U_hat * Bg)
        d32 = delta.astype(np.float32)
        A = _from_goom((K_log.real - d32) + 1j * K_log.imag)
        U = _from_goom((U_log.real + np.log(d32 + np.float32(1e-8))) + 1j * U_log.imag)
        Xh = goom_scalar_scan(A, U).astype(cdt)
    else:
        A = goom_floor(K_hat)[None, None] * np.exp(-delta)
        U = (delta + 1e-8) * goom_floor(U_hat * Bg)
        h = np.zeros_like(U[:, 0])
        hs = []
        for t in range(T):
            h = A[:, t] * h + U[:, t]
            hs.append(h)
        Xh = np.stack(hs, axis=1)
    Y_hat = Xh * Cg
    ssm = np.fft.irfft2(Y_hat, s=(H, W), axes=(3, 4)).transpose(0, 1, 3, 4, 2).astype(dtype)
    out = dense(ssm * silu(z), params["out_proj"])
    if return_intermediates:
        return out, dict(x_main=x_main, z=z, ctx=ctx, delta=delta, Bg=Bg, Cg=Cg,
                         K_hat=K_hat, ssm=ssm)
    return out


# ------------------------------------------------------------------------ GDN block
def bf16_round(a):
    """Round float values to the nearest bfloat16 (ties to even) and return them as float32:
    what `x.astype(jnp.bfloat16).astype(jnp.float32)` gives."""
    f = np.ascontiguousarray(np.asarray(a, dtype=np.float32))
    u = f.view(np.uint32)
    r = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000))
    return r.view(np.float32).reshape(f.shape)


def gdn_static_forward(params, x, *, num_timesteps, delta_key_dim=4, kernel_size=11,
                       rope_base=10000.0, spectral_rho=0.999, gate_type="factored",
                       output_norm="rms", output_gate_act="silu", use_spectral_l2_norm=True,
                       qkv_conv_size=1, no_spectral_clamp=False, carry="bf16"):
    """GatedDeltaNetCSSM static-image fast path (cssm.py:4353-4683): x is (B,H,W,C); q, k, v and
    their spectra are T-invariant, only the gates alpha_t, beta_t vary (the spatial mean of x plus
    the temporal code); the scan S_t = M_t S_{t-1} + Delta_t carries the state in the
    "linear split" bf16 format (M, Delta and the carry are rounded to bf16 real / imaginary parts,
    the products accumulate in fp32: cssm.py:4598-4632); only the final state is read out.
    Preconditions of the reference (cssm.py:4354-4370): short_conv_size=0, use_input_gates=False,
    rope_mode='none'.  carry='fp64' skips the bf16 rounding (to measure what it costs)."""
    x = np.asarray(x, np.float64)
    B, H, W, C = x.shape
    T, Wf, dk = num_timesteps, W // 2 + 1, delta_key_dim
    nh = C // dk
    W_hat = spectral_kernel(params["kernel"], H, W, spectral_rho, squash=not no_spectral_clamp)
    qkv_in = dwconv2d_same(x, params["qkv_dw"]) if qkv_conv_size > 1 else x
    qkv = dense(qkv_in, params["qkv_proj"])
    q_in, k_in, v_in = qkv[..., :C], qkv[..., C:2 * C], qkv[..., 2 * C:]
    gate_val = dense(x, params["gate_proj"])
    gate_val = silu(gate_val) if output_gate_act == "silu" else sigmoid(gate_val)

    def spec(a):
        return np.fft.rfft2(a.reshape(B, H, W, nh, dk).transpose(0, 3, 4, 1, 2), axes=(3, 4))

    q_s, k_s, v_s = spec(q_in), spec(k_in), spec(v_in)                         # (B,nh,dk,H,Wf)

    def l2(z):
        if not use_spectral_l2_norm:
            return z
        return z / np.sqrt(np.sum(np.abs(z) ** 2, axis=(3, 4), keepdims=True) + 1e-6)

    k_n = l2(k_s)
    k_n = k_n / np.sqrt(np.sum(np.abs(k_n) ** 2, axis=2, keepdims=True) + 1e-6)
    q_n = l2(q_s)
    k_outer = k_n[:, :, :, None] * np.conj(k_n[:, :, None, :])                 # (B,nh,i,j,H,Wf)
    vk_outer = v_s[:, :, :, None] * np.conj(k_n[:, :, None, :])                # (B,nh,v,j,H,Wf)

    ctx = x.mean(axis=(1, 2))[:, None, :] + temporal_ctx_code(T, C, rope_base)[None]   # (B,T,C)

    def gate(name, bounded):
        if gate_type == "factored":
            raw = sigmoid(dense(ctx, params[f"{name}_h"])[..., :, None]
                          + dense(ctx, params[f"{name}_w"])[..., None, :])
        elif gate_type == "dense":
            raw = sigmoid(dense(ctx, params[name])).reshape(B, T, H, Wf)
        else:
            raise NotImplementedError(gate_type)
        return 0.1 + 0.89 * raw if bounded else raw                            # (B,T,H,Wf)

    alpha, beta = gate("alpha", True), gate("beta", False)
    eye = np.eye(dk).reshape(1, 1, dk, dk, 1, 1)
    rnd = (lambda z: bf16_round(z.real).astype(np.float64) + 1j * bf16_round(z.imag).astype(np.float64)) \
        if carry == "bf16" else (lambda z: z)
    S = np.zeros((B, nh, dk, dk, H, Wf), dtype=np.complex128)                  # [v, i]
    for t in range(T):
        a_t = alpha[:, t][:, None, None, None]                                 # (B,1,1,1,H,Wf)
        b_t = beta[:, t][:, None, None, None]
        M = rnd(a_t * W_hat[None, :, None, None] * (eye - b_t * k_outer))      # (B,nh,i,j,H,Wf)
        D = rnd(b_t * vk_outer)                                                # (B,nh,v,j,H,Wf)
        S = rnd(np.einsum("bhijyx,bhvjyx->bhviyx", M, S) + D)
    o_hat = np.sum(S * q_n[:, :, None], axis=3).reshape(B, C, H, Wf)
    o = np.fft.irfft2(o_hat, s=(H, W), axes=(2, 3)).transpose(0, 2, 3, 1)
    if output_norm == "rms":
        o = rms_norm(o, np.asarray(params["rms_scale"], np.float64))
    elif output_norm != "none":
        raise NotImplementedError(output_norm)
    return dense(o * gate_val, params["output_proj"])


def nogate_forward(params, x, *, kernel_size, spectral_rho=0.999, dtype=np.float64):
    """NoGateCSSM.__call__ (cssm.py:6124-6175): rfft2 of the raw input, the plain complex scan
    S_t = K_hat S_{t-1} + X_hat_t (direct_scalar_scan_op: no log space, no magnitude floor),
    irfft2, Dense out_proj, minus the input."""
    cdt = np.complex128 if dtype == np.float64 else np.complex64
    x = np.asarray(x, dtype=dtype)
    B, T, H, W, C = x.shape
    K = spectral_kernel(params["kernel"], H, W, spectral_rho).astype(cdt)          # (C,H,Wf)
    U = np.fft.rfft2(x.transpose(0, 1, 4, 2, 3), axes=(3, 4)).astype(cdt)          # (B,T,C,H,Wf)
    s = np.zeros_like(U[:, 0])
    outs = []
    for t in range(T):
        s = K[None] * s + U[:, t]
        outs.append(s)
    S = np.stack(outs, axis=1)
    y = np.fft.irfft2(S, s=(H, W), axes=(3, 4)).transpose(0, 1, 3, 4, 2).astype(dtype)
    return dense(y, params["out_proj"]) - x


def additive1_forward(params, x, *, kernel_size=11, rope_mode="none", rope_base=10000.0,
                      spectral_rho=0.999, gate_type="dense", scan_mode="associative",
                      dtype=np.float64, scan="direct"):
    """AdditiveCSSM.__call__ with single_state=True (cssm.py:3061-3359, 3580-3626), gate_type
    'dense', 'factored' or 'channel', position_independent_gates=False, learned_init=False,
    use_goom=True.  With 'channel' (cssm.py:3168-3178, 3241-3244, 3615-3618) d_X is a per-channel
    scalar Dense(C)(ctx), B_X and C_gate are per-pixel maps sigmoid(Conv1x1(C)(rotated x)) applied
    in the spatial domain: x_proj * B_X before the transform, C_gate after the inverse transform.

    x_proj = Dense(C)(rope(x)); ctx = mean_{H,W}(rope(x)) + temporal code (cssm.py:3127-3131);
    d_X = 0.1 + 0.89 sigmoid(.) (bounded), B_X = C_gate = sigmoid(.), each (B,T,1,H,Wf)
    (cssm.py:3201-3207, 3224-3228); A = d_X * K_hat, U = rfft2(x_proj) * B_X (cssm.py:3282-3289);
    h_t = A_t h_{t-1} + U_t from h_0 = 0; irfft2(h * C_gate); Dense output_proj.
    scan_mode 'associative' is the log-space scan: to_goom floors the magnitudes of A and U at
    1e-7 (cssm.py:3346-3347); 'ssd' / 'quadratic' / 'pallas' evaluate the same recurrence in
    plain complex arithmetic (cssm.py:3294-3345), i.e. without the floors.
    scan='goom' (associative only) runs the literal complex64 log-space operators."""
    cdt = np.complex128 if dtype == np.float64 else np.complex64
    x = np.asarray(x, dtype=dtype)
    B, T, H, W, C = x.shape
    Wf = W // 2 + 1
    x = apply_rope(x, rope_mode, rope_base)
    x_proj = dense(x, params["x_proj"])
    ctx = x.mean(axis=(2, 3)) + temporal_ctx_code(T, C, rope_base)[None]

    chan = gate_type == "channel"

    def gate(name, bounded=False, spatial=False):
        if chan:
            if spatial:
                kern = np.asarray(params[name]["kernel"], dtype).reshape(C, C)
                return sigmoid(x @ kern + np.asarray(params[name]["bias"], dtype))     # (B,T,H,W,C)
            raw = sigmoid(dense(ctx, params[name])).reshape(B, T, C, 1, 1)
            return 0.1 + 0.89 * raw if bounded else raw
        if gate_type == "factored":
            row = dense(ctx, params[f"{name}_h"])
            col = dense(ctx, params[f"{name}_w"])
            raw = sigmoid(row[..., :, None] + col[..., None, :])
        else:
            raw = sigmoid(dense(ctx, params[name]))
        raw = raw.reshape(B, T, 1, H, Wf)
        return 0.1 + 0.89 * raw if bounded else raw

    d_X, B_X, C_gate = gate("d_X", True), gate("B_X", spatial=True), gate("C_gate", spatial=True)
    K_hat = spectral_kernel(params["kernel"], H, W, spectral_rho).astype(cdt)
    A = d_X.astype(cdt) * K_hat[None, None]
    if chan:
        U = np.fft.rfft2((x_proj * B_X).transpose(0, 1, 4, 2, 3), axes=(3, 4)).astype(cdt)
        A = np.broadcast_to(A, U.shape)
    else:
        U = np.fft.rfft2(x_proj.transpose(0, 1, 4, 2, 3), axes=(3, 4)).astype(cdt) * B_X
    if scan == "goom":
        assert scan_mode == "associative"
        V = goom_scalar_scan(A, U).astype(cdt)
    else:
        if scan_mode == "associative":
            A, U = goom_floor(A), goom_floor(U)
        h = np.zeros_like(U[:, 0])
        hs = []
        for t in range(T):
            h = A[:, t] * h + U[:, t]
            hs.append(h)
        V = np.stack(hs, axis=1)
    if chan:
        out = np.fft.irfft2(V, s=(H, W), axes=(3, 4)).transpose(0, 1, 3, 4, 2).astype(dtype) * C_gate
    else:
        out = np.fft.irfft2(V * C_gate, s=(H, W), axes=(3, 4)).transpose(0, 1, 3, 4, 2).astype(dtype)
    return dense(out, params["output_proj"])


def init_additive1_params(seed, C, H, W, *, kernel_size=11, gate_type="dense", bias_scale=0.0):
    """Parameter tree of the single-state AdditiveCSSM (cssm.py:3097, 3113, 3280-3282, 3626):
    kernel (C,ks,ks) xavier-normal, x_proj, d_X / B_X / C_gate (or their _h / _w factors),
    output_proj."""
    rng = np.random.default_rng(seed)
    Wf = W // 2 + 1
    std = np.sqrt(2.0 / (2 * kernel_size * C))          # xavier_normal on (C, ks, ks)
    p = {"kernel": (std * rng.standard_normal((C, kernel_size, kernel_size))).astype(np.float32),
         "x_proj": _dense_p(rng, C, C, bias_scale),
         "output_proj": _dense_p(rng, C, C, bias_scale)}
    for n in ("d_X", "B_X", "C_gate"):
        if gate_type == "factored":
            p[f"{n}_h"] = _dense_p(rng, C, H, bias_scale)
            p[f"{n}_w"] = _dense_p(rng, C, Wf, bias_scale)
        elif gate_type == "channel":
            d = _dense_p(rng, C, C, bias_scale)
            p[n] = d if n == "d_X" else {"kernel": d["kernel"].reshape(1, 1, C, C), "bias": d["bias"]}
        else:
            p[n] = _dense_p(rng, C, H * Wf, bias_scale)
    return p


def deltanet_forward(params, x, *, kernel_size=11, rope_mode="none", rope_base=10000.0,
                     spectral_rho=0.999, gate_type="dense", scan_mode="associative",
                     dtype=np.float64, scan="direct"):
    """DeltaNetCSSM.__call__ (cssm.py:3628-3930) for gate_type 'channel' (the default), 'dense'
    or 'factored', position_independent_gates=False, learned_init=False, use_goom=True: the
    scalar delta rule
    per channel and frequency bin,
        A_t = squash(alpha_t W_hat (1 - beta_t |k_t|^2)),  U_t = beta_t v_t conj(k_t),
        h_t = A_t h_{t-1} + U_t,  o_t = h_t q_t,
    with q, k spectrally L2-normalised per (b,t,c) (sum over the H x Wf half-spectrum bins, eps
    1e-6 under the root; k after its input gate), k and v gated by the spectral maps B_k, B_v and
    the output by C_gate (cssm.py:3756-3761, 3789-3812, 3914-3928).  With gate_type 'channel'
    alpha and beta are per-channel scalars Dense(C)(ctx) and B_k, B_v, C_gate are per-pixel,
    per-channel maps sigmoid(Conv1x1(C)(rotated x)) applied in the spatial domain: k and v
    before their transforms, C_gate after the inverse transform (cssm.py:3758-3768, 3781-3786,
    3918-3921).  scan_mode 'associative' is
    the log-space scan whose to_goom floors |A_t| and |U_t| at 1e-7 (cssm.py:3889-3890); the
    other modes run the same recurrence in plain complex arithmetic."""
    cdt = np.complex128 if dtype == np.float64 else np.complex64
    x = np.asarray(x, dtype=dtype)
    B, T, H, W, C = x.shape
    Wf = W // 2 + 1
    x = apply_rope(x, rope_mode, rope_base)
    qkv = dense(x, params["qkv_proj"])
    q_in, k_in, v_in = qkv[..., :C], qkv[..., C:2 * C], qkv[..., 2 * C:]
    ctx = x.mean(axis=(2, 3)) + temporal_ctx_code(T, C, rope_base)[None]

    def gate(name, bounded=False, spatial=False):
        if gate_type == "channel":
            if spatial:                                   # 1x1 conv, HWIO kernel (1,1,C,C)
                kern = np.asarray(params[name]["kernel"], dtype=dtype).reshape(C, C)
                return sigmoid(x @ kern + np.asarray(params[name]["bias"], dtype=dtype))
            raw = sigmoid(dense(ctx, params[name])).reshape(B, T, C, 1, 1)
            return 0.1 + 0.89 * raw if bounded else raw
        if gate_type == "factored":
            row = dense(ctx, params[f"{name}_h"])
            col = dense(ctx, params[f"{name}_w"])
            raw = sigmoid(row[..., :, None] + col[..., None, :])
        else:
            raw = sigmoid(dense(ctx, params[name]))
        raw = raw.reshape(B, T, 1, H, Wf)
        return 0.1 + 0.89 * raw if bounded else raw

    alpha, beta = gate("alpha", True), gate("beta")
    B_k, B_v, C_gate = gate("B_k", spatial=True), gate("B_v", spatial=True), gate("C_gate", spatial=True)

    def spec(z):
        return np.fft.rfft2(z.transpose(0, 1, 4, 2, 3), axes=(3, 4)).astype(cdt)

    def l2n(z):
        return z / np.sqrt(np.sum(np.abs(z) ** 2, axis=(3, 4), keepdims=True) + 1e-6)

    if gate_type == "channel":
        k_hat, v_hat, q_hat = l2n(spec(k_in * B_k)), spec(v_in * B_v), l2n(spec(q_in))
    else:
        k_hat, v_hat, q_hat = l2n(spec(k_in) * B_k), spec(v_in) * B_v, l2n(spec(q_in))
    W_hat = spectral_kernel(params["kernel"], H, W, spectral_rho).astype(cdt)[None, None]
    A = alpha * W_hat * (1.0 - beta * np.abs(k_hat) ** 2)
    A = A * spectral_rho / (1.0 + np.abs(A))
    U = beta * v_hat * np.conj(k_hat)
    if scan == "goom":
        assert scan_mode == "associative"
        h_all = goom_scalar_scan(A, U).astype(cdt)
    else:
        if scan_mode == "associative":
            A, U = goom_floor(A), goom_floor(U)
        h = np.zeros_like(U[:, 0])
        hs = []
        for t in range(T):
            h = A[:, t] * h + U[:, t]
            hs.append(h)
        h_all = np.stack(hs, axis=1)
    if gate_type == "channel":
        o = np.fft.irfft2(h_all * q_hat, s=(H, W), axes=(3, 4)).transpose(0, 1, 3, 4, 2) * C_gate
    else:
        o = np.fft.irfft2(h_all * q_hat * C_gate, s=(H, W), axes=(3, 4)).transpose(0, 1, 3, 4, 2)
    return dense(o.astype(dtype), params["output_proj"])


def init_deltanet_params(seed, C, H, W, *, kernel_size=11, gate_type="dense", bias_scale=0.0):
    """Parameter tree of DeltaNetCSSM (cssm.py:3728, 3737, 3789-3793, 3930)."""
    rng = np.random.default_rng(seed)
    Wf = W // 2 + 1
    std = np.sqrt(2.0 / (2 * kernel_size * C))
    p = {"kernel": (std * rng.standard_normal((C, kernel_size, kernel_size))).astype(np.float32),
         "qkv_proj": _dense_p(rng, C, 3 * C, bias_scale),
         "output_proj": _dense_p(rng, C, C, bias_scale)}
    for n in ("alpha", "beta", "B_k", "B_v", "C_gate"):
        if gate_type == "channel":
            p[n] = _dense_p(rng, C, C, bias_scale)
            if n in ("B_k", "B_v", "C_gate"):
                p[n]["kernel"] = p[n]["kernel"].reshape(1, 1, C, C)
        elif gate_type == "factored":
            p[f"{n}_h"] = _dense_p(rng, C, H, bias_scale)
            p[f"{n}_w"] = _dense_p(rng, C, Wf, bias_scale)
        else:
            p[n] = _dense_p(rng, C, H * Wf, bias_scale)
    return p


def rms_norm(x, w, eps=1e-6):
    """cssm.py:49-52."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def gdn_forward(params, x, *, delta_key_dim=4, kernel_size=11, rope_mode="none",
                rope_base=10000.0, spectral_rho=0.999, gate_type="factored",
                short_conv_size=4, output_norm="rms", use_input_gates=True,
                output_gate_act="silu", use_spectral_l2_norm=True, qkv_conv_size=1,
                no_spectral_clamp=False, dtype=np.float64, scan="direct",
                return_intermediates=False):
    """GatedDeltaNetCSSM.__call__, general path (cssm.py:4685-5141), for
    gate_type in {'factored','dense','channel','scalar'}, separable qkv conv, no learned_t rope, no InT
    attention, no cross-frequency conv, no SSL head.

    The reference materialises M_t (d_k x d_k) and Delta_t (d_v x d_k) per bin, repeats
    M over d_v and scans u_t = M_t u_{t-1} + Delta_t[v, :] per row v (cssm.py:4911-4958).
    scan='direct' evaluates exactly that recurrence row by row without materialising
    the repeat; scan='goom' builds the same tensors and runs the log-space operators."""
    cdt = np.complex128 if dtype == np.float64 else np.complex64
    x = np.asarray(x, dtype=dtype)
    B, T, H, W, C = x.shape
    Wf = W // 2 + 1
    dk = delta_key_dim
    dv = dk
    assert C % dk == 0
    nh = C // dk
    if gate_type not in ("factored", "dense", "channel", "scalar"):
        raise NotImplementedError(gate_type)
    x = apply_rope(x, rope_mode, rope_base)

    W_hat = spectral_kernel(params["kernel"], H, W, spectral_rho,
                            squash=not no_spectral_clamp).astype(cdt)           # (nh,H,Wf)

    xf = x.reshape(B * T, H, W, C)
    qkv_in = dwconv2d_same(xf, params["qkv_dw"]) if qkv_conv_size > 1 else xf
    qkv = dense(qkv_in, params["qkv_proj"]).reshape(B, T, H, W, 3 * C)
    q_in, k_in, v_in = qkv[..., :C], qkv[..., C:2 * C], qkv[..., 2 * C:]
    if short_conv_size > 0:
        q_in = silu(causal_tconv(q_in, params["short_conv_q"]))
        k_in = silu(causal_tconv(k_in, params["short_conv_k"]))
        v_in = silu(causal_tconv(v_in, params["short_conv_v"]))

    ctx = x.mean(axis=(2, 3)) + temporal_ctx_code(T, C, rope_base).astype(dtype)[None]

    def gate(name, bounded=False, spatial=False):
        Wd = W if spatial else Wf
        if gate_type == "channel":       # cssm.py:4800-4810: per-pixel 1x1 conv / per-head scalars
            if spatial:
                kern = params[name]["kernel"].reshape(C, C).astype(dtype)
                return sigmoid(x @ kern + params[name]["bias"].astype(dtype))      # (B,T,H,W,C)
            raw = sigmoid(dense(ctx, params[name])).reshape(B, T, nh, 1, 1)
            return 0.1 + 0.89 * raw if bounded else raw
        if gate_type == "scalar":        # cssm.py:4825-4833: one scalar per frame
            raw = sigmoid(dense(ctx, params[name])).reshape(B, T, 1, 1, 1)
            return raw if spatial or not bounded else 0.1 + 0.89 * raw
        if gate_type == "factored":
            raw = sigmoid(dense(ctx, params[f"{name}_h"])[..., :, None]
                          + dense(ctx, params[f"{name}_w"])[..., None, :])
        else:
            raw = sigmoid(dense(ctx, params[name])).reshape(B, T, H, Wd)
        if spatial:
            return raw.reshape(B, T, H, W, 1)
        raw = raw.reshape(B, T, 1, H, Wf)
        return 0.1 + 0.89 * raw if bounded else raw

    if use_input_gates:
        k_in = k_in * gate("B_k", spatial=True)
        v_in = v_in * gate("B_v", spatial=True)

    gate_val = dense(xf, params["gate_proj"]).reshape(B, T, H, W, C)
    gate_val = silu(gate_val) if output_gate_act == "silu" else sigmoid(gate_val)

    alpha = gate("alpha", bounded=True)      # (B,T,1,H,Wf)
    beta = gate("beta")

    def spec(a):
        a = a.reshape(B, T, H, W, nh, dk).transpose(0, 1, 4, 5, 2, 3)
        return np.fft.rfft2(a, axes=(4, 5)).astype(cdt)                         # (B,T,nh,dk,H,Wf)

    q_s, k_s, v_s = spec(q_in), spec(k_in), spec(v_in)

    def spectral_l2(zz):
        if not use_spectral_l2_norm:
            return zz
        return zz / np.sqrt(np.sum(np.abs(zz) ** 2, axis=(4, 5), keepdims=True) + 1e-6)

    k_s = spectral_l2(k_s)
    k_n = k_s / np.sqrt(np.sum(np.abs(k_s) ** 2, axis=3, keepdims=True) + 1e-6)
    q_n = spectral_l2(q_s)

    a_bc = alpha[:, :, :, None, None]        # (B,T,1,1,1,H,Wf)
    b_bc = beta[:, :, :, None, None]
    k_outer = k_n[:, :, :, :, None] * np.conj(k_n[:, :, :, None, :])            # [i,j]
    eye = np.eye(dk).reshape(1, 1, 1, dk, dk, 1, 1)
    M = a_bc * W_hat[None, None, :, None, None] * (eye - b_bc * k_outer)        # (B,T,nh,i,j,H,Wf)
    Delta = b_bc * (v_s[:, :, :, :, None] * np.conj(k_n[:, :, :, None, :]))     # (B,T,nh,v,j,H,Wf)

    if scan == "goom":
        M_scan = np.repeat(M.transpose(0, 1, 2, 5, 6, 3, 4), dv, axis=2)
        D_scan = Delta.transpose(0, 1, 2, 3, 5, 6, 4).reshape(B, T, nh * dv, H, Wf, dk)
        S = goom_matrix_scan(M_scan, D_scan).astype(cdt)
        S = S.reshape(B, T, nh, dv, H, Wf, dk)
    else:
        Mf = goom_floor(M)
        Df = goom_floor(Delta)
        s = np.zeros((B, nh, dv, dk, H, Wf), dtype=cdt)        # [v,i]
        Ss = []
        for t in range(T):
            s = np.einsum("bhijyx,bhvjyx->bhviyx", Mf[:, t], s) + Df[:, t]
            Ss.append(s)
        S = np.stack(Ss, axis=1).transpose(0, 1, 2, 3, 5, 6, 4)                 # (B,T,nh,v,H,Wf,i)
    o_hat = np.sum(S * q_n.transpose(0, 1, 2, 4, 5, 3)[:, :, :, None], axis=-1)
    o_hat = o_hat.reshape(B, T, C, H, Wf)
    o = np.fft.irfft2(o_hat, s=(H, W), axes=(3, 4)).transpose(0, 1, 3, 4, 2).astype(dtype)
    pre_norm = o
    if output_norm == "rms":
        o = rms_norm(o, params["rms_scale"].astype(dtype))
    elif output_norm != "none":
        raise NotImplementedError(output_norm)
    out = dense(o * gate_val, params["output_proj"])
    if return_intermediates:
        return out, dict(q_in=q_in, k_in=k_in, v_in=v_in, gate_val=gate_val, ctx=ctx,
                         alpha=alpha, beta=beta, W_hat=W_hat, o_spatial=pre_norm)
    return out


# ------------------------------------------------------------- seeded weight trees
def _lecun(rng, shape, fan_in):
    return (rng.standard_normal(shape) / np.sqrt(fan_in)).astype(np.float32)


def _dense_p(rng, cin, cout, bias_scale):
    return {"kernel": _lecun(rng, (cin, cout), cin),
            "bias": (bias_scale * rng.standard_normal(cout)).astype(np.float32)}


def init_gated_params(seed, C, H, W, *, kernel_size, gate_type="dense", short_conv_size=4,
                      short_conv_spatial_size=3, bias_scale=0.0):
    """NumPy-seeded stand-ins for the Flax initialisers, with the reference's parameter
    names and shapes (cssm.py:481-584).  `bias_scale` > 0 gives non-zero biases (zeros,
    the Flax default, would hide bias indexing mistakes)."""
    rng = np.random.default_rng(seed)
    Wf = W // 2 + 1
    p = {"in_proj": _dense_p(rng, C, 2 * C, bias_scale),
         "kernel": (0.02 * rng.standard_normal((C, kernel_size, kernel_size))).astype(np.float32),
         "out_proj": _dense_p(rng, C, C, bias_scale)}
    if short_conv_spatial_size > 0:
        k = short_conv_spatial_size
        p["short_conv_spatial"] = {"kernel": _lecun(rng, (k, k, 1, C), k * k),
                                   "bias": (bias_scale * rng.standard_normal(C)).astype(np.float32)}
    if short_conv_size > 0:
        k = short_conv_size
        p["short_conv_temporal"] = {"kernel": _lecun(rng, (k, 1, C), k),
                                    "bias": (bias_scale * rng.standard_normal(C)).astype(np.float32)}
    for n in ("delta_proj", "B_proj", "C_proj"):
        if gate_type == "factored":
            p[f"{n}_h"] = _dense_p(rng, C, H, bias_scale)
            p[f"{n}_w"] = _dense_p(rng, C, Wf, bias_scale)
        else:
            p[n] = _dense_p(rng, C, H * Wf, bias_scale)
    return p


def init_gdn_params(seed, C, H, W, *, delta_key_dim=4, kernel_size=11, gate_type="factored",
                    short_conv_size=4, qkv_conv_size=1, use_input_gates=True,
                    bias_scale=0.0, perturb_rms=False):
    """Parameter tree of GatedDeltaNetCSSM (cssm.py:4729-5141)."""
    rng = np.random.default_rng(seed)
    Wf = W // 2 + 1
    nh = C // delta_key_dim
    std = np.sqrt(2.0 / (2 * kernel_size * nh))       # xavier_normal on (nh, ks, ks)
    p = {"kernel": (std * rng.standard_normal((nh, kernel_size, kernel_size))).astype(np.float32),
         "qkv_proj": _dense_p(rng, C, 3 * C, bias_scale),
         "gate_proj": _dense_p(rng, C, C, bias_scale),
         "output_proj": _dense_p(rng, C, C, bias_scale),
         "rms_scale": np.ones(C, np.float32)}
    if perturb_rms:
        p["rms_scale"] = (1.0 + 0.2 * rng.standard_normal(C)).astype(np.float32)
    if qkv_conv_size > 1:
        k = qkv_conv_size
        p["qkv_dw"] = {"kernel": _lecun(rng, (k, k, 1, C), k * k),
                       "bias": (bias_scale * rng.standard_normal(C)).astype(np.float32)}
    if short_conv_size > 0:
        k = short_conv_size
        for n in ("short_conv_q", "short_conv_k", "short_conv_v"):
            p[n] = {"kernel": _lecun(rng, (k, 1, C), k),
                    "bias": (bias_scale * rng.standard_normal(C)).astype(np.float32)}
    names = [("alpha", Wf), ("beta", Wf)]
    if use_input_gates:
        names += [("B_k", W), ("B_v", W)]
    for n, wd in names:
        if gate_type == "factored":
            p[f"{n}_h"] = _dense_p(rng, C, H, bias_scale)
            p[f"{n}_w"] = _dense_p(rng, C, wd, bias_scale)
        elif gate_type == "channel":
            if n.startswith("B_"):
                d = _dense_p(rng, C, C, bias_scale)
                p[n] = {"kernel": d["kernel"].reshape(1, 1, C, C), "bias": d["bias"]}
            else:
                p[n] = _dense_p(rng, C, nh, bias_scale)
        elif gate_type == "scalar":
            p[n] = _dense_p(rng, C, 1, bias_scale)
        else:
            p[n] = _dense_p(rng, C, H * wd, bias_scale)
    return p


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
