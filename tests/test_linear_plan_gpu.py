"""Launch plan (next-launch L2 prefetch): a recorded sequence of linears gives bit-identical results with the
hints on, in every later round, and a call outside the recorded order only switches the hints off."""
import numpy as np
import pytest
import torch

from conftest import synth_linear

pytestmark = pytest.mark.gpu


def _layer(cuda, seed):
    """Four projections in the order of one decoder layer: fused qkv-like, o, gate/up SwiGLU, down."""
    shapes = {"qkv": (1024, 2048 + 256 + 256), "o": (2048, 1024), "ffn": (1024, 2816), "down": (2816, 1024)}
    w = {}
    for i, (name, (K, N)) in enumerate(shapes.items()):
        _, W, S, _ = synth_linear(1, K, N, seed=seed + i)
        w[name] = (torch.from_numpy(W).cuda(), torch.from_numpy(S).cuda(), K, N)
    _, Wu, Su, _ = synth_linear(1, 1024, 2816, seed=seed + 9)
    w["up"] = (torch.from_numpy(Wu).cuda(), torch.from_numpy(Su).cuda(), 1024, 2816)
    return w


def _run(cuda, w, X, M):
    Wq, Sq, K, N = w["qkv"]
    yq = torch.empty((M, 2048), dtype=torch.float16, device="cuda")
    yk = torch.empty((M, 256), dtype=torch.float16, device="cuda")
    yv = torch.empty((M, 256), dtype=torch.float16, device="cuda")
    cuda.linear_int4_fused(X, [dict(Y=yq, W_int4=Wq[:2048], scales=Sq[:2048], bias=None, N=2048),
                               dict(Y=yk, W_int4=Wq[2048:2304], scales=Sq[2048:2304], bias=None, N=256),
                               dict(Y=yv, W_int4=Wq[2304:], scales=Sq[2304:], bias=None, N=256)], M, K)
    Wo, So, Ko, No = w["o"]
    yo = torch.empty((M, No), dtype=torch.float16, device="cuda")
    cuda.linear_int4(yo, yq, Wo, So, None, M, No, Ko)
    Wg, Sg, Kg, Ng = w["ffn"]
    Wu, Su, _, _ = w["up"]
    ym = torch.empty((M, Ng), dtype=torch.float16, device="cuda")
    cuda.mlp_gate_up_swiglu_int4(ym, yo, Wg, Sg, Wu, Su, M, Ng, Kg)
    Wd, Sd, Kd, Nd = w["down"]
    yd = torch.empty((M, Nd), dtype=torch.float16, device="cuda")
    cuda.linear_int4(yd, ym, Wd, Sd, None, M, Nd, Kd)
    torch.cuda.synchronize()
    return [t.clone() for t in (yq, yk, yv, yo, ym, yd)]


@pytest.mark.parametrize("M", [1, 8, 32])
def test_plan_does_not_change_results(cuda, M):
    w = _layer(cuda, seed=100 + M)
    X = (torch.randn((M, 1024), device="cuda") * 0.5).half()
    plan = cuda.LinearPlan()
    plan.clear()
    base = _run(cuda, w, X, M)                      # no plan
    with plan.record():
        rec = _run(cuda, w, X, M)                   # recording round
    for a, b in zip(base, rec):
        assert torch.equal(a, b)
    for _ in range(3):                              # hinted rounds
        plan.rewind()
        got = _run(cuda, w, X, M)
        for a, b in zip(base, got):
            assert torch.equal(a, b)
    assert cuda.device_status(0) == 0
    # a call that is not in the recorded order: still correct, hints go off, later rounds still correct
    plan.rewind()
    Wd, Sd, Kd, Nd = w["down"]
    y = torch.empty((M, Nd), dtype=torch.float16, device="cuda")
    cuda.linear_int4(y, base[4], Wd, Sd, None, M, Nd, Kd)
    torch.cuda.synchronize()
    assert torch.equal(y, base[5])
    got = _run(cuda, w, X, M)
    for a, b in zip(base, got):
        assert torch.equal(a, b)
    plan.clear()
    assert cuda.device_status(0) == 0
