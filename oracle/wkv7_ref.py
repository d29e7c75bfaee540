"""TEST INFRASTRUCTURE — torch restatement of the reference's per-op fp32 references.

Nothing in the shipped package imports this file.  Each function restates the
in-file reference the upstream test scripts compare their kernels against, so
that the parity tests here read like the upstream ones:

  ref_attn          wind_rwkv/rwkv7/time_mixer.py:6-16, tests/test_attn.py:6-18
                    (extended: optional s0 in, optional sT out — same loop body)
  ref_attn_ln       tests/test_attn_ln.py:6-21
  ref_ddlerp        tests/test_ddlerp.py:5-13
  ref_expand_loras  tests/test_expand_loras.py:6-19 (upstream reads B,T,C from
                    module globals; here they come from the input shape)
  ref_time_mixer    tests/test_time_mixer.py:13-55 (RefTimeMixer.forward) as a
                    function of a parameter dict

All accept any float dtype; computation runs in `compute_dtype` (fp32 as
upstream, or fp64 for measuring rounding floors) and gradients come from
autograd through these loops.
"""
import torch as th

F = th.nn.functional


def ref_attn(q, w, k, v, a, b, HEAD_SIZE, s0=None, return_state=False, compute_dtype=th.float32):
    dtype = w.dtype
    B, T, HC = q.shape
    H, C = HC // HEAD_SIZE, HEAD_SIZE
    q, w, k, v, a, b = [i.view(B, T, H, C).to(compute_dtype) for i in [q, w, k, v, a, b]]
    s = th.zeros(B, H, C, C, device=q.device, dtype=compute_dtype) if s0 is None else s0.to(compute_dtype)
    w = th.exp(-th.exp(w))
    ys = []
    for t in range(T):
        s = s * w[:, t, :, None, :] + s @ a[:, t, :, :, None] * b[:, t, :, None, :] + v[:, t, :, :, None] * k[:, t, :, None, :]
        ys.append((s @ q[:, t, :, :, None]).squeeze(-1))
    y = th.stack(ys, dim=1).to(dtype).view(B, T, HC)
    return (y, s) if return_state else y


def ref_attn_ln(q, w, k, v, a, b, g, params, HEAD_SIZE, s0=None, return_state=False, compute_dtype=th.float32):
    dtype = w.dtype
    B, T, HC = q.shape
    H, C = HC // HEAD_SIZE, HEAD_SIZE
    cd = compute_dtype
    y, s = ref_attn(q.to(cd), w.to(cd), k.to(cd), v.to(cd), a.to(cd), b.to(cd), HEAD_SIZE, s0, True, cd)
    q, k, v, g = [i.view(B, T, H, C).to(cd) for i in [q, k, v, g]]
    params = params.to(cd)
    y = F.group_norm(y.view(B * T, HC), H, params[0], params[1], eps=64e-5).view(B, T, H, C)
    y = y + (q * k * params[2].view(H, C)).sum(dim=-1, keepdim=True) * v
    y = (y * g).view(B, T, HC).to(dtype)
    return (y, s) if return_state else y


def ref_ddlerp(x, mix_x, Wmix1, Wmix2, mix_bias, compute_dtype=th.float32):
    B, T, C = x.shape
    dtype = x.dtype
    x, mix_x, Wmix1, Wmix2, mix_bias = [i.to(compute_dtype) for i in [x, mix_x, Wmix1, Wmix2, mix_bias]]
    xx = F.pad(x, (0, 0, 1, -1)) - x
    xxx = x + xx * mix_x
    xxx = th.tanh(xxx @ Wmix1.mT).view(B * T, 4, -1).transpose(0, 1)
    xxx = (xxx @ Wmix2.mT).view(4, B, T, C)
    return (x + xx * (xxx + mix_bias)).to(dtype).unbind(dim=0)


def ref_expand_loras(w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias,
                     HEAD_SIZE, compute_dtype=th.float32, out_dtype=th.bfloat16):
    B, T, C = w_in.shape
    w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias = [
        i.to(compute_dtype) for i in [w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias]]
    w_out = -F.softplus(-(w_bias + w_in)) - 0.5
    z = k_in + th.tanh(z_in) @ Wz.mT
    z_out = F.normalize(z.view(B, T, -1, HEAD_SIZE), dim=-1, p=2.0).view(B, T, C)
    a = th.sigmoid(a_bias + a_in @ Wa.mT)
    ma = th.sigmoid(ma_bias + ma_in @ Wma.mT)
    k = k_in * ma + k_in * a * (1 - ma)
    mk = th.sigmoid(mk_bias + mk_in @ Wmk.mT)
    k_out = k * (w_out * mk).exp()
    b_out = -z_out * a
    return tuple(i.to(out_dtype) for i in [w_out, k_out, z_out, b_out])


def ref_time_mixer(p, x, n_head, compute_dtype=th.float32):
    """RefTimeMixer.forward with parameters taken from dict `p` (names as upstream's TimeMixer)."""
    cd = compute_dtype
    p = {n: t.to(cd) for n, t in p.items()}
    x = x.to(cd)
    B, T, C = x.shape
    H = n_head
    xx = F.pad(x, (0, 0, 1, -1)) - x
    xxx = x + xx * p['time_maa_x']
    xxx = th.tanh(xxx @ p['time_maa_w1'].mT).view(B * T, 4, -1).transpose(0, 1)
    xxx = (xxx @ p['time_maa_w2'].mT).view(4, B, T, -1)
    xrg, xwa, xk, xv = (x + xx * (xxx + p['time_maa'])).unbind(dim=0)
    r = xrg @ p['Wr'].mT
    w = -F.softplus(-(p['time_decay'] + th.tanh(xwa @ p['time_decay_w1'].mT) @ p['time_decay_w2'].mT)) - 0.5
    k = xk @ p['Wk'].mT
    v = xv @ p['Wv'].mT
    g = th.tanh(xrg @ p['gate_w1'].mT) @ p['gate_w2'].mT
    kk = k + th.tanh(xk @ p['time_kkk_w1'].mT) @ p['time_kkk_w2'].mT
    kk = F.normalize(kk.view(B, T, H, -1), dim=-1, p=2.0).view(B, T, C)
    a = th.sigmoid(p['time_aaaaa'] + (xwa @ p['time_aaa_w1'].mT) @ p['time_aaa_w2'].mT)
    ma = th.sigmoid(p['time_misc_a'] + (xwa @ p['ma_w1'].mT) @ p['ma_w2'].mT)
    k = k * ma + k * a * (1 - ma)
    mk = th.sigmoid(p['time_misc_k'] + (xk @ p['mk_w1'].mT) @ p['mk_w2'].mT)
    k = k * th.clamp(w * mk, max=0).exp()
    x = ref_attn(r, w, k, v, -kk, kk * a, C // H, compute_dtype=cd)
    x = F.group_norm(x.view(B * T, C), H, p['ln_x.weight'], p['ln_x.bias'], eps=64e-5).view(B, T, C)
    x = x + ((r.view(B, T, H, -1) * k.view(B, T, H, -1) * p['time_faaaa'].view(H, -1)).sum(dim=-1, keepdim=True) * v.view(B, T, H, -1)).view(B, T, C)
    return (x * g) @ p['Wo'].mT
