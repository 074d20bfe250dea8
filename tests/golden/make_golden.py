"""Generates the golden fixtures of this directory by running the reference
project's own Python code on CPU.

Run from the repository root in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/nnue-pytorch

The fixtures (*.npz, a few hundred KB in total) are committed; the test suite
only reads them, so it runs where the reference checkout does not exist.
Two tiny stand-ins let `import model` work without optional packages the
reference imports at module scope: `chess` (only piece constants and a
`Piece(type, color)` record are used, for initial PSQT values) and
`torchmetrics` (running means of the loss); `numba`, when absent, is replaced
by an identity `njit` decorator (the reference's LEB128 loops then run as
plain Python).
"""

from __future__ import annotations

import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def install_shims():
    chess = types.ModuleType("chess")
    chess.PAWN, chess.KNIGHT, chess.BISHOP, chess.ROOK, chess.QUEEN, chess.KING = 1, 2, 3, 4, 5, 6
    chess.WHITE, chess.BLACK = True, False

    class Piece:
        def __init__(self, piece_type, color):
            self.piece_type, self.color = piece_type, color

    chess.Piece = Piece
    sys.modules["chess"] = chess

    tm = types.ModuleType("torchmetrics")

    class MeanMetric(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.total, self.n = 0.0, 0

        def update(self, v):
            self.total += float(v)
            self.n += 1

        def compute(self):
            return torch.tensor(self.total / max(self.n, 1))

        def reset(self):
            self.total, self.n = 0.0, 0

    class MetricCollection(torch.nn.ModuleDict):
        pass

    tm.MeanMetric, tm.MetricCollection = MeanMetric, MetricCollection
    sys.modules["torchmetrics"] = tm


def to_np(d):
    return {k: (v.detach().cpu().numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in d.items()}


def main(ref_root: str):
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))  # repo root (positions generator)
    sys.path.insert(0, ref_root)
    install_shims()
    torch.set_num_threads(4)

    sl = importlib.import_module("model.modules.feature_transformer.sparse_linear_functions")
    dft = importlib.import_module("model.modules.feature_transformer.double_ft_functions")
    hk = importlib.import_module("model.modules.features.halfka_v2_hm")
    rl = importlib.import_module("model.optimizers.ranger_lite")
    import chess
    import model as ref_model
    from model.config import ModelConfig, NNUELightningConfig
    from model.nnue import NNUE, calculate_sf_loss
    from model.config import LossParams
    from model.quantize import QuantizationConfig

    from nnue_pytorch_b200 import positions

    # 1. sparse linear, the shapes of the reference's tests/test_feature_transformer.py
    g = torch.Generator().manual_seed(0)
    w = torch.rand(10, 128, generator=g)
    b = torch.rand(128, generator=g)
    idx = (torch.rand(16, 32, generator=g) * 10).to(torch.int32)
    idx[3, 20:] = -1
    idx[7, :] = -1
    go = torch.randn(16, 128, generator=g)
    wr, br = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    out = sl.SparseLinearFunction.apply(idx, wr, br, "torch")
    (out * go).sum().backward()
    np.savez_compressed(os.path.join(HERE, "sparse_linear.npz"), **to_np(
        dict(weight=w, bias=b, indices=idx, grad_out=go, out=out, grad_weight=wr.grad, grad_bias=br.grad)))

    # 2. fused double FT, the shapes of tests/test_fused_double_ft.py (l1 = 32) and a 0/1 side-to-move
    #    case with the trainer's activation cap, where the clamp is active on both sides
    for name, l1, randn_stm, max_act, wscale in (("fused_ft_randn", 32, True, 127.0, 1.0),
                                                  ("fused_ft_stm", 256, False, 255.0 / 256.0, 0.25)):
        g = torch.Generator().manual_seed(1)
        B, K, N, P = 6, 32, 100, 8
        us = torch.randn(B, 1, generator=g) if randn_stm else torch.randint(0, 2, (B, 1), generator=g).float()
        them = torch.randn(B, 1, generator=g) if randn_stm else 1.0 - us
        wi = torch.randint(0, N, (B, K), generator=g, dtype=torch.int32)
        bi = torch.randint(0, N, (B, K), generator=g, dtype=torch.int32)
        wi[:, -2:] = -1
        bi[:, -2:] = -1
        wi[1, 5:] = -1
        bi[2, :] = -1
        ps = torch.randint(0, P, (B,), generator=g, dtype=torch.int64)
        w = torch.randn(N, l1 + P, generator=g) * wscale
        b = torch.randn(l1 + P, generator=g) * wscale
        gl0 = torch.randn(B, l1, generator=g)
        gwp = torch.randn(B, 1, generator=g)
        gbp = torch.randn(B, 1, generator=g)
        wr, br = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
        l0, wp, bp = dft.double_feature_transform(us, them, wi, bi, ps, wr, br, max_act, l1, "torch")
        ((l0 * gl0).sum() + (wp * gwp).sum() + (bp * gbp).sum()).backward()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **to_np(dict(
            us=us, them=them, white=wi, black=bi, psqt=ps, weight=w, bias=b, max_act=max_act, l1=l1,
            grad_l0=gl0, grad_wpsqt=gwp, grad_bpsqt=gbp,
            l0=l0, wpsqt=wp, bpsqt=bp, grad_weight=wr.grad, grad_bias=br.grad)))

    # 3. HalfKAv2_hm index formula on generated positions
    pos = positions.generate_positions(64, 5)
    exp_w = np.full((64, 32), -1, np.int32)
    exp_b = np.full((64, 32), -1, np.int32)
    for i in range(64):
        for s in range(int(pos.piece_count[i])):
            piece = chess.Piece(int(pos.piece_type[i, s]), bool(pos.is_white[i, s]))
            exp_w[i, s] = hk._halfka_idx(True, int(pos.squares[i, 0]), int(pos.squares[i, s]), piece)
            exp_b[i, s] = hk._halfka_idx(False, int(pos.squares[i, 1]), int(pos.squares[i, s]), piece)
    np.savez_compressed(os.path.join(HERE, "halfka_indices.npz"), white=exp_w, black=exp_b,
                        king_buckets=np.asarray(hk.KingBuckets, np.int64),
                        psqt_init=np.asarray(hk.HalfKav2Hm.halfka_psqts(), np.int64))

    # 4. RangerLite, Python path: 12 steps on three tensors, default trainer settings and a decayed variant
    for name, wd in (("ranger_lite", 0.0), ("ranger_lite_wd", 0.01)):
        g = torch.Generator().manual_seed(2)
        shapes = [(40, 24), (24,), (7, 5)]
        ps = [torch.nn.Parameter(torch.randn(*s, generator=g) * 0.1) for s in shapes]
        init = [p.detach().clone() for p in ps]
        opt = rl.RangerLite([{"params": [ps[0]], "lr": 8.75e-4, "weight_decay": wd},
                             {"params": ps[1:], "lr": 8.75e-4, "weight_decay": 0.0}],
                            lr=1.0, weight_decay=0.0, use_legacy_scoping_bug=False, normloss_active=False,
                            pnm_activate=True, pnm_momentum=1.0, lookahead_blending_alpha=0.5, lookahead_mergetime=5)
        rec = {}
        for j, p0 in enumerate(init):
            rec[f"init{j}"] = p0
        for step in range(12):
            for j, p in enumerate(ps):
                gr = torch.randn(*shapes[j], generator=g) * 0.05
                if j == 0:
                    gr[::3] = 0.0  # rows that never receive gradient
                p.grad = gr
                rec[f"grad{step}_{j}"] = gr.clone()
            opt.step()
            for j, p in enumerate(ps):
                rec[f"param{step}_{j}"] = p.detach().clone()
        for j, p in enumerate(ps):
            st = opt.state[p]
            rec[f"grad_ma{j}"], rec[f"neg_grad_ma{j}"] = st["grad_ma"], st["neg_grad_ma"]
            rec[f"variance_ma{j}"], rec[f"slow{j}"] = st["variance_ma"], st["lookahead_params"]
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **to_np(rec))

    # 5. whole model: float32 training loss + gradients, float64 fake-quantized forward (the exact
    #    definition of the quantized evaluation), native HalfKAv2_hm^ layout, L1 = 64
    cfg = NNUELightningConfig(features="HalfKAv2_hm^", model_config=ModelConfig(L1=64, L2=32, L3=32))
    torch.manual_seed(3)
    nnue = NNUE(cfg)
    m = nnue.model
    gen = np.random.default_rng(11)
    with torch.no_grad():
        # grid-aligned, in-range weights so the integer restatement sees the same numbers
        m.input.features[0].weight.copy_(torch.from_numpy(gen.integers(-40, 41, (24576, 72)) / 256.0))
        m.input.features[0].weight[:, 64:] = torch.from_numpy(gen.integers(-3000, 3001, (24576, 8)) / 9600.0)
        m.input.features[0].virtual_weight.copy_(torch.from_numpy(gen.integers(-20, 21, (768, 72)) / 256.0))
        m.input.features[0].virtual_weight[:, 64:] = torch.from_numpy(gen.integers(-900, 901, (768, 8)) / 9600.0)
        m.input.bias[:64] = torch.from_numpy(gen.integers(-60, 61, 64) / 256.0)
        m.layer_stacks.l1.linear.weight.copy_(torch.from_numpy(gen.integers(-90, 91, (256, 64)) / 128.0))
        m.layer_stacks.l1.factorized_linear.weight.copy_(torch.from_numpy(gen.integers(-30, 31, (32, 64)) / 128.0))
        m.layer_stacks.l1.linear.bias.copy_(torch.from_numpy(gen.integers(-9000, 9001, 256) / 16384.0))
        m.layer_stacks.l1.factorized_linear.bias.copy_(torch.from_numpy(gen.integers(-3000, 3001, 32) / 16384.0))
        m.layer_stacks.l2.linear.weight.copy_(torch.from_numpy(gen.integers(-100, 101, (256, 64)) / 64.0))
        m.layer_stacks.l2.linear.bias.copy_(torch.from_numpy(gen.integers(-6000, 6001, 256) / 8192.0))
        m.layer_stacks.output.linear.weight.copy_(torch.from_numpy(gen.integers(-120, 121, (8, 128)) / 128.0))
        m.layer_stacks.output.linear.bias.copy_(torch.from_numpy(gen.integers(-9000, 9001, 8) / 16384.0))
    batch = positions.generate_batch(96, 21, layout="native")
    tb = tuple(torch.from_numpy(a) for a in batch.as_tuple())
    nnue.train()
    loss = nnue.train_step(tb, 0, 0)["loss"]
    loss.backward()
    rec = dict(loss=loss.detach(),
               g_ft_weight=m.input.features[0].weight.grad, g_ft_virtual=m.input.features[0].virtual_weight.grad,
               g_ft_bias=m.input.bias.grad, g_l1_w=m.layer_stacks.l1.linear.weight.grad,
               g_l1f_w=m.layer_stacks.l1.factorized_linear.weight.grad, g_out_w=m.layer_stacks.output.linear.weight.grad)
    with torch.no_grad():
        y32 = m(tb[0], tb[1], tb[2], tb[3], tb[6], True, True)
        md = ref_model.NNUEModel("HalfKAv2_hm^", ModelConfig(L1=64, L2=32, L3=32)).double()
        md.load_state_dict({k: v.double() for k, v in m.state_dict().items()})
        y64 = md(tb[0].double(), tb[1].double(), tb[2], tb[3], tb[6], True, True)
    rec.update(scorenet32=y32, eval_int=torch.round(y64 * 19200).to(torch.int64), seed_pos=21, seed_w=11)
    np.savez_compressed(os.path.join(HERE, "model_small.npz"), **to_np(rec))

    # 6. loss function alone, including tablebase-range scores
    g = torch.Generator().manual_seed(4)
    sn = torch.randn(64, 1, generator=g) * 500
    sc = torch.randn(64, 1, generator=g) * 700
    sc[:4, 0] = torch.tensor([31990.0, -31900.0, 31800.0, -31756.0])
    oc = torch.randint(0, 3, (64, 1), generator=g).float() * 0.5
    vals = [calculate_sf_loss(sn, sc, oc, LossParams(), lam) for lam in (1.0, 0.6)]
    np.savez_compressed(os.path.join(HERE, "sf_loss.npz"), scorenet=sn.numpy(), score=sc.numpy(), outcome=oc.numpy(),
                        loss_lambda_1=vals[0].numpy(), loss_lambda_06=vals[1].numpy())
    # 7. `.nnue` file of the model of section 5, written by the reference's own serializer
    #    (a few MB: only its SHA-256, length and first bytes are kept)
    import hashlib

    if "numba" not in sys.modules:
        try:
            import numba  # noqa: F401
        except ImportError:  # the reference only uses numba.njit, as a plain decorator
            nb = types.ModuleType("numba")
            nb.njit = lambda f: f
            sys.modules["numba"] = nb
    ser = importlib.import_module("model.utils.serialize")
    rec = {}
    with torch.no_grad():
        for comp in ("none", "leb128"):
            data = bytes(ser.NNUEWriter(m, ft_compression=comp, verbose=False).buf)
            rec[f"sha256_{comp}"] = np.frombuffer(hashlib.sha256(data).digest(), dtype=np.uint8)
            rec[f"length_{comp}"] = len(data)
            rec[f"head_{comp}"] = np.frombuffer(data[:1024], dtype=np.uint8)
            rec[f"tail_{comp}"] = np.frombuffer(data[-1024:], dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "nnue_file.npz"), **rec)

    # 8. index lists of the default feature set on real positions: the reference loader's own extractors
    #    (compiled here from its sources, where they lie) over every 23rd entry of its sample binpack
    import subprocess
    import tempfile

    binpack = os.path.join(ref_root, ".pgo", "small.binpack")
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "dump_features")
        subprocess.run(["g++", "-std=c++20", "-O1", "-I" + os.path.join(ref_root, "data_loader", "cpp"),
                        os.path.join(HERE, "dump_features.cpp"), "-o", exe, "-lpthread"], check=True)
        text = subprocess.run([exe, binpack, "300", "23"], check=True, capture_output=True, text=True).stdout
    rows = [list(map(int, ln.split())) for ln in text.strip().splitlines()]
    n = len(rows)
    boards = np.zeros((n, 64), np.int8)
    stm = np.zeros(n, np.int8)
    lists = {name: np.full((n, 2, k), -1, np.int32) for name, k in (("halfka", 32), ("threats", 128), ("pawn_pairs", 128))}
    for i, v in enumerate(rows):
        boards[i], stm[i], at = v[:64], v[64], 65
        for side in range(2):
            for name in ("halfka", "threats", "pawn_pairs"):
                k = v[at]
                lists[name][i, side, :k] = v[at + 1 : at + 1 + k]
                at += 1 + k
        assert at == len(v)
    np.savez_compressed(os.path.join(HERE, "full_features.npz"), boards=boards, black_to_move=stm, **lists)

    _ = QuantizationConfig
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/nnue-pytorch")
    main(sys.argv[1])
