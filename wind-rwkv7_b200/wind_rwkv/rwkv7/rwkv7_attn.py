"""WKV7 attention: drop-in for wind_rwkv/rwkv7/rwkv7_attn.py of johanwind/wind-rwkv7.

Same entry points and argument order (`load_attn(HEAD_SIZE)`, `attn(r,w,k,v,a,b,HEAD_SIZE)`,
`WindRWKV7.apply(w,q,k,v,a,b,s0) -> (y, sT, s)`); the work is done by the sm_100a kernels of
libwkv7_sm100.so.  Differences, all additive: states and chunk checkpoints are fp32 (upstream:
bf16), float32 tensors are accepted as well as bfloat16, `attn` takes keyword-only `s0` and
`return_state`, and launches go to the current stream.
"""
import torch as th

from . import _lib


def _same_layout(ts):
    s = ts[0].stride()
    return all(t.stride() == s and t.stride(3) == 1 for t in ts)


def fw_attn(w, q, k, v, a, b, s0, save_checkpoints=True):
    """Forward launcher (upstream: rwkv7_attn.py:5-11). Returns y, sT (fp32), s (fp32 checkpoints).
    With save_checkpoints=False (no backward will follow) the checkpoint tensor is empty and the
    kernel skips its stores."""
    B, T, H, C = w.shape
    _lib.require_cuda(w, q, k, v, a, b, s0)
    if not _same_layout([w, q, k, v, a, b]):
        w, q, k, v, a, b = [i.contiguous() for i in (w, q, k, v, a, b)]
    y = th.empty_like(v)
    if y.stride() != v.stride():
        y = th.empty_strided(v.shape, v.stride(), dtype=v.dtype, device=v.device)
    sT = th.empty(B, H, C, C, dtype=th.float32, device=w.device)
    s = th.empty(B, H, _lib.chunks(T) if save_checkpoints else 0, _lib.CKPT_FLOATS, dtype=th.float32, device=w.device)
    sb, st, sh = _lib.strides4(w)
    with _lib.on_device(w, q, k, v, a, b, s0):
        rc = _lib.lib().wkv7_fwd(q.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
                                 _lib.ptr(s0), y.data_ptr(), sT.data_ptr(), s.data_ptr() if save_checkpoints else None,
                                 B, T, H, C, sb, st, sh, _lib.io_dtype(w), _lib.stream_of(w))
    _lib.check(rc, 'wkv7_fwd')
    return y, sT, s


def bw_attn(w, q, k, v, a, b, s, dy, dsT, sT):
    """Backward launcher (upstream: rwkv7_attn.py:13-16)."""
    B, T, H, C = w.shape
    if not _same_layout([w, q, k, v, a, b, dy]):
        w, q, k, v, a, b, dy = [i.contiguous() for i in (w, q, k, v, a, b, dy)]
    dw, dq, dk, dv, da, db = [th.empty_strided(w.shape, w.stride(), dtype=w.dtype, device=w.device) for _ in range(6)]
    ds0 = th.empty(B, H, C, C, dtype=th.float32, device=w.device)
    sb, st, sh = _lib.strides4(w)
    with _lib.on_device(w, q, k, v, a, b, s, dy, dsT):
        rc = _lib.lib().wkv7_bwd(q.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
                                 dy.data_ptr(), s.data_ptr(), _lib.ptr(dsT), _lib.ptr(sT if dsT is not None else None),
                                 dq.data_ptr(), dw.data_ptr(), dk.data_ptr(), dv.data_ptr(), da.data_ptr(), db.data_ptr(),
                                 ds0.data_ptr(), B, T, H, C, sb, st, sh, _lib.io_dtype(w), _lib.stream_of(w))
    _lib.check(rc, 'wkv7_bwd')
    return dw, dq, dk, dv, da, db, ds0


def _fake_fw(w, q, k, v, a, b, s0, save_checkpoints=True):
    B, T, H, C = w.shape
    return (th.empty_like(v), w.new_empty((B, H, C, C), dtype=th.float32),
            w.new_empty((B, H, _lib.chunks(T) if save_checkpoints else 0, _lib.CKPT_FLOATS), dtype=th.float32))


def _fake_bw(w, q, k, v, a, b, s, dy, dsT, sT):
    B, T, H, C = w.shape
    return tuple(th.empty_like(w) for _ in range(6)) + (w.new_empty((B, H, C, C), dtype=th.float32),)


_fw_op = _lib.opaque_op('attn_fwd', fw_attn, _fake_fw,
                        '(Tensor w, Tensor q, Tensor k, Tensor v, Tensor a, Tensor b, Tensor? s0, bool save_checkpoints=True) -> (Tensor, Tensor, Tensor)')
_bw_op = _lib.opaque_op('attn_bwd', bw_attn, _fake_bw,
                        '(Tensor w, Tensor q, Tensor k, Tensor v, Tensor a, Tensor b, Tensor s, Tensor dy, Tensor? dsT, Tensor sT) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)')


def _check_inputs(w, q, k, v, a, b, s0):
    B, T, H, C = w.shape
    assert C == _lib.HEAD_SIZE, 'only head size 64 is built'
    assert all(i.dtype == w.dtype for i in [q, k, v, a, b]), 'r,w,k,v,a,b must share one dtype'
    assert all(i.shape == w.shape for i in [q, k, v, a, b])
    if s0 is not None:
        assert list(s0.shape) == [B, H, C, C]


class WindRWKV7(th.autograd.Function):
    """(w,q,k,v,a,b,s0) -> (y, sT, s), as upstream's autograd function (rwkv7_attn.py:18-44).

    s0 may be None (zeros), fp32, or bf16 (converted); sT and ds0 are fp32 unless s0 was bf16.
    """

    @staticmethod
    def forward(ctx, w, q, k, v, a, b, s0):
        if not th.compiler.is_compiling():  # as upstream, checks are skipped while tracing
            _check_inputs(w, q, k, v, a, b, s0)
        s0f = None if s0 is None else s0.float().contiguous()
        save = True if th.compiler.is_compiling() else any(ctx.needs_input_grad)
        y, sT, s = _lib.call(_fw_op, fw_attn, w, q, k, v, a, b, s0f, save)
        ctx.save_for_backward(w, q, k, v, a, b, s, sT)
        ctx.s0_dtype = None if s0 is None else s0.dtype
        ctx.mark_non_differentiable(s)
        ctx.set_materialize_grads(False)
        if s0 is not None and s0.dtype != th.float32:
            return y, sT.to(s0.dtype), s
        return y, sT, s

    @staticmethod
    def backward(ctx, dy, dsT, ds):
        w, q, k, v, a, b, s, sT = ctx.saved_tensors
        if not th.compiler.is_compiling():
            assert ds is None
        if dy is None:
            dy = th.zeros_like(v)
        if dsT is not None:
            dsT = dsT.float().contiguous()
        dw, dq, dk, dv, da, db, ds0 = _lib.call(_bw_op, bw_attn, w, q, k, v, a, b, s, dy, dsT, sT)
        if ctx.s0_dtype is None:
            ds0 = None
        elif ctx.s0_dtype != th.float32:
            ds0 = ds0.to(ctx.s0_dtype)
        return dw, dq, dk, dv, da, db, ds0


def load_attn(HEAD_SIZE):
    """Upstream JIT-compiles its extension here (rwkv7_attn.py:46-51); this loads the prebuilt library."""
    if HEAD_SIZE != _lib.HEAD_SIZE:
        raise ValueError(f'only HEAD_SIZE == {_lib.HEAD_SIZE} is built, got {HEAD_SIZE}')
    _lib.lib()


def _attn_time_split(r, w, k, v, a, b, C, s0, nseg):
    """Forward only, the sequence cut into `nseg` equal segments that run as separate chains (for B*H far below the
    number of SMs: one CTA walks one chain, so a single long sequence otherwise occupies H SMs).

    The recurrence is affine in the state: over a segment S_end = S_start M + R, with M and R independent of S_start.
    Pass 1 runs every segment twice (two concurrent launches of nseg*B*H chains): from the zero state with the real inputs
    (final state = R) and from the identity state with v = 0 (final state = M).  A short host loop of nseg - 1 batched
    64x64 products gives every segment's start state; pass 2 is the ordinary forward over the segments with those.
    Three passes of length T/nseg instead of one of length T.  Results differ from the unsplit call by the rounding
    of M (single-TF32 products for bf16 tensors): y and sT agree within the path's tolerance, not bit for bit."""
    B, T, HC = w.shape
    H = HC // C
    assert T % nseg == 0, 'time_split must divide T'
    Ts = T // nseg
    ins = [i.contiguous().view(B * nseg, Ts, H, C) for i in (w, r, k, v, a, b)]   # segments become batch entries: no copy
    dev = w.device
    eye = th.eye(C, dtype=th.float32, device=dev).expand(B * nseg, H, C, C)
    zero = th.zeros(B * nseg, H, C, C, dtype=th.float32, device=dev)
    # the two sets of chains read the same inputs (v apart): two launches on two streams, which share the SMs
    side = th.cuda.Stream(dev)
    main = th.cuda.current_stream(dev)
    side.wait_stream(main)
    with th.cuda.stream(side):
        insM = list(ins)
        insM[3] = th.zeros_like(ins[3])                                           # v = 0 for the identity chains
        _, M, _ = fw_attn(*insM, eye.contiguous(), save_checkpoints=False)
    _, R, _ = fw_attn(*ins, zero, save_checkpoints=False)
    main.wait_stream(side)
    for t in insM + [M]:
        t.record_stream(main)
    R, M = R.view(B, nseg, H, C, C), M.view(B, nseg, H, C, C)
    S = th.zeros(B, H, C, C, dtype=th.float32, device=dev) if s0 is None else s0.float()
    starts = [S]
    prev = th.backends.cuda.matmul.allow_tf32
    th.backends.cuda.matmul.allow_tf32 = False
    try:
        for j in range(nseg - 1):
            S = S @ M[:, j] + R[:, j]
            starts.append(S)
    finally:
        th.backends.cuda.matmul.allow_tf32 = prev
    y, sT, _ = fw_attn(*ins, th.stack(starts, 1).reshape(B * nseg, H, C, C).contiguous(), save_checkpoints=False)
    return y.view(B, T, HC), sT.view(B, nseg, H, C, C)[:, -1].contiguous()


def _fw_into(w, q, k, v, a, b, s0, y):
    """Forward without checkpoints into a caller-provided y view that shares the inputs' strides. Returns sT."""
    B, T, H, C = w.shape
    assert _same_layout([w, q, k, v, a, b, y]), 'inputs and output must share one layout'
    sT = th.empty(B, H, C, C, dtype=th.float32, device=w.device)
    sb, st, sh = _lib.strides4(w)
    with _lib.on_device(w, q, k, v, a, b, s0):
        rc = _lib.lib().wkv7_fwd(q.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
                                 _lib.ptr(s0), y.data_ptr(), sT.data_ptr(), None, B, T, H, C, sb, st, sh,
                                 _lib.io_dtype(w), _lib.stream_of(w))
    _lib.check(rc, 'wkv7_fwd')
    return sT


def tail_split_plan(B, T, H, sms):
    """(number of chains cut in time, segments) for attn(..., time_split='tail'), or None when it does not pay.

    One CTA walks one chain, so B*H chains take ceil(B*H / sms) rounds of T steps; the last round runs
    B*H mod sms chains and leaves the other SMs idle.  Those chains (they must lie within the last batch entry)
    can instead run as n segments each through the affine form (three passes of T/n steps)."""
    chains = B * H
    tail = chains % sms
    if chains <= sms or tail == 0 or tail > H:
        return None
    # Cost of the three passes in time steps of one chain: 3 passes x rounds of SMs x (segment length + a chain's start-up,
    # about 300 steps) + the n - 1 serial start-state products (about 250 steps' worth each: two small launches).
    # Worth it below the one round of T steps that it replaces (measured on B200: T = 16384, 12 chains: n = 8 is
    # the fastest of 4 / 8 / 16 / 32, as this model says).
    best = None
    for n in range(4, 33):
        if T % n or (T // n) % 16:
            continue
        cost = 3 * -(-tail * n // sms) * (T // n + 300) + (n - 1) * 250
        if best is None or cost < best[0]:
            best = (cost, n)
    return (tail, best[1]) if best and best[0] < 0.85 * T else None


_TAIL_STREAMS = {}


def _tail_streams(dev):
    """Two side streams per device, the second of high priority, created once: libraries keep per-stream state (a BLAS
    handle and its workspace), and a fresh stream on every call would pay for that state again and again."""
    key = th.device(dev).index if th.device(dev).index is not None else th.cuda.current_device()
    if key not in _TAIL_STREAMS:
        _TAIL_STREAMS[key] = [th.cuda.Stream(dev), th.cuda.Stream(dev, priority=-1)]
    return _TAIL_STREAMS[key]


def _attn_tail_split(r, w, k, v, a, b, C, s0):
    """Forward only.  All chains but those of the last, partly filled round of SMs run as usual; the rest are cut in
    time (see tail_split_plan and _attn_time_split; here M comes from a pass that starts at the identity state with
    the real inputs, S_end = M + R, so no zero copy of v is needed).  The three groups of launches go to three
    streams, write into views of one output tensor (head slices of the last batch entry, no copies) and share the
    SMs.  Falls back to the plain call when the shape gives no such tail."""
    B, T, HC = w.shape
    H = HC // C
    dev = w.device
    plan = tail_split_plan(B, T, H, th.cuda.get_device_properties(dev).multi_processor_count)
    ins = [i.contiguous().view(B, T, H, C) for i in (w, r, k, v, a, b)]
    y = th.empty(B, T, H, C, dtype=w.dtype, device=dev)
    s0 = None if s0 is None else s0.float().contiguous()
    if plan is None:
        sT = _fw_into(*ins, s0, y)
        return y.view(B, T, HC), sT
    tail, n = plan
    h0, Ts = H - tail, T // n
    sT = th.empty(B, H, C, C, dtype=th.float32, device=dev)
    main = th.cuda.current_stream(dev)
    # the short chains go first and on a high-priority stream, so that their dependent passes are not queued behind
    # the long chains' second round
    sides = _tail_streams(dev)
    for sd in sides:
        sd.wait_stream(main)
    with th.cuda.stream(sides[1]):
        # segments of the last entry's remaining heads as batch entries: [n, Ts, tail, C] views, no copy
        def seg(x):
            return x.as_strided((n, Ts, tail, C), (Ts * HC, HC, C, 1), x[B - 1, 0, h0, 0].storage_offset())
        sin, sy = [seg(i) for i in ins], seg(y)
        eye = th.eye(C, dtype=th.float32, device=dev).expand(n, tail, C, C).contiguous()
        R = _fw_into(*sin, None, sy)
        M = _fw_into(*sin, eye, sy) - R
        S = th.zeros(tail, C, C, dtype=th.float32, device=dev) if s0 is None else s0[B - 1, h0:]
        starts = [S]
        prev = th.backends.cuda.matmul.allow_tf32
        th.backends.cuda.matmul.allow_tf32 = False
        try:
            for j in range(n - 1):
                S = S @ M[j] + R[j]
                starts.append(S)
        finally:
            th.backends.cuda.matmul.allow_tf32 = prev
        sT[B - 1, h0:] = _fw_into(*sin, th.stack(starts, 0).contiguous(), sy)[-1]
    if B > 1:  # whole batch entries
        sT[:B - 1] = _fw_into(*[i[:B - 1] for i in ins], None if s0 is None else s0[:B - 1].contiguous(), y[:B - 1])
    if h0 > 0:  # the last entry's heads that still fit the full rounds
        with th.cuda.stream(sides[0]):
            sT[B - 1:, :h0] = _fw_into(*[i[B - 1:, :, :h0] for i in ins], None if s0 is None else s0[B - 1:, :h0].contiguous(), y[B - 1:, :, :h0])
    for sd in sides:
        main.wait_stream(sd)
    for t in ins + [y, sT] + ([] if s0 is None else [s0]):
        for sd in sides:
            t.record_stream(sd)
    return y.view(B, T, HC), sT


def attn(r, w, k, v, a, b, HEAD_SIZE, *, s0=None, return_state=False, time_split=None):
    """y = WKV7(r,w,k,v,a,b) for [B,T,H*HEAD_SIZE] tensors (upstream: rwkv7_attn.py:53-59).

    time_split=n (no upstream counterpart; inference only, no autograd): the sequence runs as n segments in
    parallel, see _attn_time_split.  Pays when B*H is far below the number of SMs.
    time_split='tail': only the chains of the last, partly filled round of SMs are cut in time, see _attn_tail_split."""
    B, T, HC = w.shape
    C = HEAD_SIZE
    H = HC // C
    if time_split == 'tail' or (time_split is not None and time_split > 1):
        assert C == _lib.HEAD_SIZE, 'only head size 64 is built'
        assert not (th.is_grad_enabled() and any(i.requires_grad for i in (r, w, k, v, a, b))), 'time_split is forward only'
        if time_split == 'tail':
            y, sT = _attn_tail_split(r, w, k, v, a, b, C, s0)
        else:
            y, sT = _attn_time_split(r, w, k, v, a, b, C, s0, int(time_split))
        return (y, sT) if return_state else y
    r, w, k, v, a, b = [i.view(B, T, H, C) for i in [r, w, k, v, a, b]]
    y, sT, _ = WindRWKV7.apply(w, r, k, v, a, b, s0)
    y = y.view(B, T, HC)
    return (y, sT) if return_state else y


def attn_step(r, w, k, v, a, b, HEAD_SIZE, state=None, *, inplace=False):
    """Decode: advances the recurrence over the T (typically 1) time steps of [B,T,H*HEAD_SIZE] tensors.

    Returns (y, new_state).  `state` is the fp32 [B,H,HEAD_SIZE,HEAD_SIZE] state `attn(..., return_state=True)`
    returns (None = zeros); with inplace=True it is overwritten and returned.  No autograd, no checkpoints.
    Upstream has no counterpart; this is the loop body of its naive recurrence (time_mixer.py:13-15) as a kernel."""
    B, T, HC = w.shape
    C = HEAD_SIZE
    H = HC // C
    assert C == _lib.HEAD_SIZE, 'only head size 64 is built'
    _lib.require_cuda(r, w, k, v, a, b, state)
    r, w, k, v, a, b = [i.contiguous().view(B, T, H, C) for i in [r, w, k, v, a, b]]
    assert all(i.dtype == w.dtype for i in [r, k, v, a, b]), 'r,w,k,v,a,b must share one dtype'
    if state is not None:
        assert state.dtype == th.float32 and list(state.shape) == [B, H, C, C] and state.is_contiguous()
    y = th.empty_like(v)
    sT = state if (inplace and state is not None) else th.empty(B, H, C, C, dtype=th.float32, device=w.device)
    sb, st, sh = _lib.strides4(w)
    with _lib.on_device(r, w, k, v, a, b, state):
        rc = _lib.lib().wkv7_step(r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
                                  _lib.ptr(state), y.data_ptr(), sT.data_ptr(), B, T, H, C, sb, st, sh,
                                  _lib.io_dtype(w), _lib.stream_of(w))
    _lib.check(rc, 'wkv7_step')
    return y.view(B, T, HC), sT
