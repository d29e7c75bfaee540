"""RWKV-7 time mixer: drop-in for wind_rwkv/rwkv7/time_mixer.py (`TimeMixer(args, layer_id, ...)`,
`ref_attn`).  Same parameter names, shapes and initial distributions as upstream (time_mixer.py:19-104),
so state dicts are interchangeable; the forward (upstream :106-167) composes the sm_100a ops of this
package (ddlerp -> projections -> expand_loras -> attn_ln -> output projection).  Dense projections
are plain bf16 matmuls (cuBLAS), as upstream.

Only one backend exists here.  `use_triton_ddlerp`, `use_triton_loras` and `triton_dot_prec` are
accepted for signature compatibility and ignored; `attn_impl` must be 'cuda'.
"""
import torch
import torch.nn as nn

from .rwkv7_attn_ln import attn_ln, load_attn_ln
from .rwkv7_ddlerp import ddlerp
from .rwkv7_expand_loras import expand_loras
from .rwkv7_proj import proj as fused_proj


class _CastAll(torch.autograd.Function):
    """bf16 copies of the projection weights in one multi-tensor copy, and their gradients back to the parameters'
    dtypes in another (upstream casts weight by weight, time_mixer.py:120-131: a dozen small launches each way)."""

    @staticmethod
    def forward(ctx, *params):
        ctx.dtypes = [p.dtype for p in params]
        outs = [torch.empty_like(p, dtype=torch.bfloat16) for p in params]
        torch._foreach_copy_(outs, [p.detach() for p in params])
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        idx = [i for i, g in enumerate(grads) if g is not None]
        outs = [torch.empty_like(grads[i], dtype=ctx.dtypes[i]) for i in idx]
        if idx:
            torch._foreach_copy_(outs, [grads[i].contiguous() for i in idx])
        res = [None] * len(grads)
        for i, o in zip(idx, outs):
            res[i] = o
        return tuple(res)


def ref_attn(q, w, k, v, a, b, HEAD_SIZE):
    """The naive per-step recurrence (upstream time_mixer.py:6-16), kept for users who call it to
    check results; it runs on whatever device and dtype its inputs have."""
    B, T, HC = q.shape
    H, C = HC // HEAD_SIZE, HEAD_SIZE
    q, w, k, v, a, b = [i.view(B, T, H, C) for i in [q, w, k, v, a, b]]
    state = torch.zeros(B, H, C, C, device=q.device, dtype=q.dtype)
    decay = torch.exp(-torch.exp(w))
    out = []
    for t in range(T):
        sa = state @ a[:, t, :, :, None]
        state = state * decay[:, t, :, None, :] + sa * b[:, t, :, None, :] + v[:, t, :, :, None] * k[:, t, :, None, :]
        out.append((state @ q[:, t, :, :, None]).squeeze(-1))
    return torch.stack(out, dim=1).view(B, T, HC)


def _orthogonal(shape, scale):
    """Orthogonal init with upstream's gain rule: sqrt(rows/cols) when rows > cols, applied per
    matrix for 3-d shapes."""
    x = torch.zeros(shape)
    mats = [x] if x.dim() == 2 else list(x)
    for m in mats:
        rows, cols = m.shape
        nn.init.orthogonal_(m, gain=(max(rows / cols, 1.0) ** 0.5) * scale)
    return x


class TimeMixer(nn.Module):
    MIX_RANK, DECAY_RANK, SMALL_RANK, GATE_RANK = 32, 64, 16, 128

    def __init__(self, args, layer_id, use_triton_ddlerp=True, use_triton_loras=True, attn_impl='cuda', triton_dot_prec='fp32'):
        super().__init__()
        if attn_impl != 'cuda':
            raise ValueError("only attn_impl='cuda' exists in this build (no Triton or PyTorch-loop backend)")
        self.args, self.layer_id = args, layer_id
        C = self.n_embd = self.dim_att = args.n_embd
        self.n_head = args.n_head
        assert C % self.n_head == 0
        self.head_size = C // self.n_head
        load_attn_ln(self.head_size)

        depth = layer_id / max(args.n_layer - 1, 1)      # 0 at the first layer, 1 at the last
        shallow = 1.0 - layer_id / args.n_layer          # 1 at the first layer, towards 0 at the last
        pos = torch.arange(C) / C

        def mix(power, shift=0.0):
            return 1.0 - (torch.pow(pos, power * shallow) + shift * depth)

        self.time_maa_x = nn.Parameter(1.0 - torch.pow(pos, 0.6 * shallow ** 0.9))
        self.time_maa = nn.Parameter(torch.stack([mix(0.2), mix(0.9), mix(0.9, 0.4), mix(0.4, 0.6)])[:, None, None, :])
        ramp = torch.arange(C) / (C - 1)
        self.time_decay = nn.Parameter(-7 + 5 * ramp ** (0.85 + depth ** 0.5) + 0.5)   # +0.5: the softplus offset
        self.time_faaaa = nn.Parameter(torch.zeros(C))
        self.time_aaaaa = nn.Parameter(torch.zeros(C))

        r = self.SMALL_RANK
        self.time_maa_w1 = nn.Parameter(torch.zeros(4 * self.MIX_RANK, C))
        self.time_maa_w2 = nn.Parameter(_orthogonal((4, self.MIX_RANK, C), 0.1).mT.contiguous())
        self.time_decay_w1 = nn.Parameter(torch.zeros(self.DECAY_RANK, C))
        self.time_decay_w2 = nn.Parameter(_orthogonal((self.DECAY_RANK, C), 0.1).mT.contiguous())
        self.time_aaa_w1 = nn.Parameter(torch.zeros(r, C))
        self.time_aaa_w2 = nn.Parameter(_orthogonal((r, C), 0.1).mT.contiguous())
        self.time_kkk_w1 = nn.Parameter(torch.zeros(r, C))
        self.time_kkk_w2 = nn.Parameter(_orthogonal((r, C), 0.1).mT.contiguous())
        self.gate_w1 = nn.Parameter(_orthogonal((self.GATE_RANK, C), 0.1))
        self.gate_w2 = nn.Parameter(_orthogonal((self.GATE_RANK, C), 0.1).mT.contiguous())
        self.ma_w1 = nn.Parameter(torch.zeros(r, C))
        self.ma_w2 = nn.Parameter(_orthogonal((r, C), 0.1).mT.contiguous())
        self.time_misc_a = nn.Parameter(torch.zeros(C))
        self.mk_w1 = nn.Parameter(torch.zeros(r, C))
        self.mk_w2 = nn.Parameter(_orthogonal((r, C), 0.1).mT.contiguous())
        self.time_misc_k = nn.Parameter(torch.zeros(C))

        def uniform(scale):
            bound = scale / C ** 0.5
            return nn.Parameter(torch.empty(C, C).uniform_(-bound, bound))

        self.Wr, self.Wk, self.Wv, self.Wo = uniform(0.5), uniform(0.05), uniform(0.5), uniform(0)
        self.ln_x = nn.GroupNorm(self.n_head, C, eps=64e-5)

    # the weights of the plain projections (their gradients are bf16 products anyway); the parameters of ddlerp and
    # expand_loras go to those ops as they are: the ops cast them themselves and return fp32 gradients
    _BF16_PARAMS = ('Wr', 'Wk', 'Wv', 'Wo', 'gate_w1', 'gate_w2', 'time_kkk_w1', 'mk_w1', 'time_decay_w1', 'time_aaa_w1', 'ma_w1',
                    'time_decay_w2')

    def forward(self, x):
        r16 = self.SMALL_RANK
        bf = torch.bfloat16
        P = dict(zip(self._BF16_PARAMS, _CastAll.apply(*[getattr(self, n) for n in self._BF16_PARAMS])))  # bf16, one launch
        xrg, xwa, xk, xv = ddlerp(x.to(bf), self.time_maa_x, self.time_maa_w1, self.time_maa_w2, self.time_maa)

        def proj(inp, name):
            return inp @ P[name].mT

        def lora1(inp, tanh_cols, *names):
            # first stage of one or several LoRAs on the tcgen05 projection kernel, tanh fused into the chosen columns
            return fused_proj(inp, torch.cat([P[n] for n in names]) if len(names) > 1 else P[names[0]], tanh_cols)

        r = proj(xrg, 'Wr')
        g = lora1(xrg, (0, self.GATE_RANK), 'gate_w1') @ P['gate_w2'].mT
        k = proj(xk, 'Wk')
        kk1, mk1 = lora1(xk, None, 'time_kkk_w1', 'mk_w1').split([r16, r16], dim=2)
        v = proj(xv, 'Wv')
        w1t, a1, ma1 = lora1(xwa, (0, self.DECAY_RANK), 'time_decay_w1', 'time_aaa_w1', 'ma_w1').split(
            [self.DECAY_RANK, r16, r16], dim=2)
        w2 = w1t @ P['time_decay_w2'].mT

        w, k, kk, b = expand_loras(w2, k, kk1, a1, ma1, mk1, self.time_kkk_w2, self.time_aaa_w2, self.ma_w2, self.mk_w2,
                                   self.time_decay, self.time_aaaaa, self.time_misc_a, self.time_misc_k, self.head_size)
        params = torch.stack([self.ln_x.weight, self.ln_x.bias, self.time_faaaa]).float()
        y = attn_ln(r, w, k, v, kk, b, g, params, self.head_size)
        return y @ P['Wo'].mT
