"""GPU parity of the fused RangerLite update against the golden fixtures (made
by the reference's own optimizer) and the CPU oracle."""

import pytest
import torch

from _util import load_golden, max_rel_err, t

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return torch.device("cuda:0")


def _make(params, wd0, **kw):
    from nnue_pytorch_b200.ranger_lite import RangerLite

    return RangerLite(
        [{"params": [params[0]], "lr": 8.75e-4, "weight_decay": wd0},
         {"params": params[1:], "lr": 8.75e-4, "weight_decay": 0.0}],
        lr=1.0, weight_decay=0.0, use_legacy_scoping_bug=False, normloss_active=False, pnm_activate=True,
        pnm_momentum=1.0, lookahead_blending_alpha=0.5, lookahead_mergetime=5, **kw)


@pytest.mark.parametrize("name,wd", [("ranger_lite", 0.0), ("ranger_lite_wd", 0.01)])
def test_matches_reference_steps(dev, name, wd):
    g = load_golden(name)
    params = [torch.nn.Parameter(t(g[f"init{j}"]).to(dev)) for j in range(3)]
    opt = _make(params, wd)
    for step in range(12):
        for j, p in enumerate(params):
            p.grad = t(g[f"grad{step}_{j}"]).to(dev)
        opt.step()
        for j, p in enumerate(params):
            ref = t(g[f"param{step}_{j}"])
            assert max_rel_err(p.detach().cpu(), ref) <= 1e-6, (name, step, j)
    for j, p in enumerate(params):
        st = opt.state[p]
        for key, gk in (("grad_ma", "grad_ma"), ("neg_grad_ma", "neg_grad_ma"), ("variance_ma", "variance_ma"),
                        ("lookahead_params", "slow")):
            assert max_rel_err(st[key].cpu(), t(g[f"{gk}{j}"])) <= 1e-5, (name, key, j)
    assert set(opt.state[params[0]].keys()) >= {"step", "grad_ma", "variance_ma", "neg_grad_ma", "lookahead_params"}


def test_touched_rows_only_is_bit_identical(dev):
    """A 2-D table large enough for the row-skipping kernel: same bits as the
    flat kernel, rows without gradient never change, and a row touched once
    keeps being updated afterwards (momentum)."""
    gen = torch.Generator().manual_seed(0)
    rows, width = 2048, 264
    init = torch.randn(rows, width, generator=gen) * 0.1
    pa = torch.nn.Parameter(init.clone().to(dev))
    pb = torch.nn.Parameter(init.clone().to(dev))
    oa = _make([pa, torch.nn.Parameter(torch.zeros(4, device=dev))], 0.0, touched_rows_only=True)
    ob = _make([pb, torch.nn.Parameter(torch.zeros(4, device=dev))], 0.0, touched_rows_only=False)
    never = torch.zeros(rows, dtype=torch.bool)
    never[::5] = True
    for step in range(11):
        gr = torch.randn(rows, width, generator=gen) * 0.05
        gr[never] = 0.0
        if step >= 3:
            gr[1::5] = 0.0  # touched during the first steps, silent afterwards
        pa.grad = gr.to(dev)
        pb.grad = gr.to(dev)
        oa.step()
        ob.step()
        assert torch.equal(pa.detach(), pb.detach()), step
    assert torch.equal(pa.detach().cpu()[never], init[never])
    assert not torch.equal(pa.detach().cpu()[1::5], init[1::5])
    flags = oa._row_active[id(pa)].cpu().bool()
    assert torch.equal(flags, ~never)
    for key in ("grad_ma", "neg_grad_ma", "variance_ma", "lookahead_params"):
        assert torch.equal(oa.state[pa][key], ob.state[pb][key]), key


def test_oracle_parity_over_many_steps(dev):
    """25 steps (five lookahead merges) against the CPU oracle, with the clip
    coefficient folded in through `grad_scale`."""
    from oracle import ranger_lite_oracle

    gen = torch.Generator().manual_seed(5)
    shapes = [(1500, 72), (72,), (256, 64), (256,), (8, 128), (8,)]
    init = [torch.randn(*s, generator=gen) * 0.1 for s in shapes]
    cpu = [x.clone() for x in init]
    st = ranger_lite_oracle.RangerLiteState(cpu)
    params = [torch.nn.Parameter(x.clone().to(dev)) for x in init]
    opt = _make(params, 0.0)
    scale = torch.tensor([0.37], device=dev)
    opt.grad_scale = scale
    for step in range(25):
        grads = [torch.randn(*s, generator=gen) * 0.02 for s in shapes]
        grads[0][::4] = 0.0
        ranger_lite_oracle.ranger_lite_step(cpu, [g * 0.37 for g in grads], st, lr=8.75e-4)
        for p, g in zip(params, grads):
            p.grad = g.to(dev)
        opt.step()
    for p, c in zip(params, cpu):
        assert max_rel_err(p.detach().cpu(), c) <= 1e-5


def test_eval_train_swap_and_state_dict_round_trip(dev):
    gen = torch.Generator().manual_seed(6)
    p = torch.nn.Parameter((torch.randn(64, 16, generator=gen)).to(dev))
    q = torch.nn.Parameter(torch.zeros(3, device=dev))
    opt = _make([p, q], 0.0)
    for _ in range(3):
        p.grad = torch.randn(64, 16, generator=gen).to(dev)
        q.grad = torch.randn(3, generator=gen).to(dev)
        opt.step()
    fast = p.detach().clone()
    slow = opt.state[p]["lookahead_params"].clone()
    opt.eval()
    assert torch.equal(p.detach(), slow)
    opt.eval()  # idempotent
    assert torch.equal(p.detach(), slow)
    opt.train()
    assert torch.equal(p.detach(), fast)
    import copy

    sd = copy.deepcopy(opt.state_dict())  # a checkpoint holds its own tensors
    p2 = torch.nn.Parameter(p.detach().clone())
    q2 = torch.nn.Parameter(q.detach().clone())
    opt2 = _make([p2, q2], 0.0)
    opt2.load_state_dict(sd)
    g1 = torch.randn(64, 16, generator=gen).to(dev)
    p.grad, p2.grad = g1, g1.clone()
    q.grad, q2.grad = torch.ones(3, device=dev), torch.ones(3, device=dev)
    opt2.lookahead_step = opt.lookahead_step  # the merge counter is not part of the state dict
    opt.step()
    opt2.step()
    assert torch.equal(p.detach(), p2.detach())


def test_clip_coefficient_matches_torch(dev):
    from nnue_pytorch_b200 import _launch

    gen = torch.Generator().manual_seed(7)
    gs = [torch.randn(1000, 77, generator=gen).to(dev), torch.randn(13, generator=gen).to(dev)]
    sumsq = torch.zeros(1, device=dev)
    coef = torch.zeros(1, device=dev)
    for g in gs:
        _launch.grad_sumsq(g, sumsq)
    for max_norm in (2.0, 1e6):
        _launch.clip_coef(sumsq, max_norm, coef)
        total = torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(g) for g in gs]))
        want = torch.clamp(max_norm / (total + 1e-6), max=1.0)
        assert abs(float(coef) - float(want)) <= 1e-5 * float(want)
        # gradients that are sums over 4 ranks: the same clip on their mean, times 1/4
        _launch.clip_coef(sumsq, max_norm, coef, 0.25)
        want = 0.25 * torch.clamp(max_norm / (0.25 * total + 1e-6), max=1.0)
        assert abs(float(coef) - float(want)) <= 1e-5 * float(want)


def test_multi_tensor_norm_matches_per_tensor_calls(dev):
    from nnue_pytorch_b200 import _launch

    gen = torch.Generator().manual_seed(9)
    shapes = [(3072,), (32, 3072), (32,), (256, 3072), (256,), (256, 64), (256,), (8, 128), (8,), (5001, 264), (3,)] * 2
    gs = [torch.randn(*sh, generator=gen).to(dev) for sh in shapes]  # 22 tensors: more than one launch's worth
    gs.append(torch.randn(17, generator=gen).to(dev)[1:])             # not 16-byte aligned
    multi = torch.zeros(1, device=dev)
    _launch.grad_sumsq_multi(gs, multi)
    want = sum(float((g.double() ** 2).sum()) for g in gs)
    assert abs(float(multi) - want) <= 1e-5 * want
    _launch.grad_sumsq_multi([], multi)  # nothing to add
    assert abs(float(multi) - want) <= 1e-5 * want


def test_multi_tensor_update_is_bitwise_the_single_tensor_update(dev):
    """Nine small tensors with different constants in one launch = nine launches."""
    from nnue_pytorch_b200 import _launch

    gen = torch.Generator().manual_seed(4)
    shapes = [(3080,), (32, 3072), (32,), (256, 3072), (255,), (256, 64), (7,), (8, 128), (1,)]

    def state():
        g2 = torch.Generator().manual_seed(5)
        out = []
        for sh in shapes:
            out.append([torch.randn(*sh, generator=g2).to(dev) * s for s in (0.1, 0.01, 0.02, 0.02)] +
                       [torch.rand(*sh, generator=g2).to(dev) * 1e-3, torch.randn(*sh, generator=g2).to(dev) * 0.1])
        return out  # p, grad, grad_ma, neg_grad_ma, variance_ma, slow

    scale = torch.full((1,), 0.37, device=dev)
    for step_no, merge in ((1, 0), (2, 0), (5, 1)):
        hps = []
        for i in range(len(shapes)):
            hps.append(_launch.hparams_struct(
                beta2=0.999, one_minus_beta2=0.001, mom=0.81, one_minus_mom=0.19, one_plus_f=2.0, f=1.0,
                noise_norm_inv=5.0 ** -0.5, step_size=8.75e-4 * (1 + 0.1 * i), bc2_sqrt=(1 - 0.999 ** step_no) ** 0.5,
                eps=1e-7, wd_keep=1.0 if i % 2 else 0.999, alpha=0.5, one_minus_alpha=0.5, use_pnm=1,
                step_is_odd=step_no % 2, do_merge=merge, phase=0))
        a, b = state(), state()
        for (p, g, gm, ngm, vm, slow), hp in zip(a, hps):
            _launch.ranger_update(p, g, gm, ngm, vm, slow, None, scale, hp)
        _launch.ranger_update_multi([(p, g, gm, ngm, vm, slow, hp) for (p, g, gm, ngm, vm, slow), hp in zip(b, hps)], scale)
        for ta, tb in zip(a, b):
            for x, y in zip(ta, tb):
                assert torch.equal(x, y), (step_no, x.shape)
    _ = gen
