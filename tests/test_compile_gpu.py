"""torch.compile(fullgraph=True) keeps working through the ops, as upstream's own scripts use them
(tests/test_ddlerp.py:37, tests/test_expand_loras.py:57, tests/test_attn_ln.py:52): compiled
forward+backward must equal the eager result (the same kernels run): bit for bit, except for the
weight gradients of ddlerp and expand_loras, whose fp32 atomic accumulation order varies from run to
run (relative difference below 1e-5)."""
import pytest
import torch as th

pytestmark = pytest.mark.gpu


def test_compiled_ops_match_eager():
    from wind_rwkv.rwkv7 import attn_ln, ddlerp, expand_loras, synthetic
    from test_ddlerp_gpu import data as ddlerp_data
    from test_expand_loras_gpu import data as loras_data
    N, B, T, H = 64, 2, 64, 2
    d = synthetic.wkv7_inputs(B, T, H, N, seed=30, dtype=th.bfloat16, device='cuda')
    g, params = synthetic.attn_ln_extras(B, T, H, N, seed=30, dtype=th.bfloat16, device='cuda')
    cases = {
        'attn_ln': (lambda *a: attn_ln(*a, N), [d[n] for n in 'rwkvab'] + [g, params]),
        'ddlerp': (ddlerp, [ddlerp_data(B, T, 128, 16, 31)[0].cuda()] + [i.float().cuda() for i in ddlerp_data(B, T, 128, 16, 31)[1:]]),
        'expand_loras': (lambda *a: expand_loras(*a, N), [i.cuda() for i in loras_data(B, T, 128, 16, 32)[:6]] +
                         [i.float().cuda() for i in loras_data(B, T, 128, 16, 32)[6:]]),
    }
    for name, (f, ins) in cases.items():
        def run(fn):
            xs = [i.detach().clone().requires_grad_() for i in ins]
            out = fn(*xs)
            outs = out if isinstance(out, tuple) else (out,)
            th.manual_seed(0)
            th.autograd.backward(outs, [th.randn_like(o) for o in outs])
            return [o.detach() for o in outs] + [x.grad for x in xs]
        eager = run(f)
        compiled = run(th.compile(f, fullgraph=True))
        for i, (a, b) in enumerate(zip(eager, compiled)):
            same = th.equal(a, b) or float((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-30)) < 1e-5
            assert same, f'{name}: tensor {i} differs between eager and compiled'
