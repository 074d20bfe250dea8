"""Integer evaluation of a quantized net, restated on numpy int64.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

The reference project has no integer evaluator: its "quantized evaluation" is
the float forward with fake quantization switched on
(model/quantize.py:36-56,133-147, model/modules/layer_stacks.py:33-84,
model/model.py:107-133).  Run in float64 that forward is exact, and
`integer_eval` below is the same arithmetic on integers:

  acc = Bq + sum Wq[idx] per perspective, side to move first; c = clamp(acc, 0, 255)
  x0  = [(c0*c1) >> 9, (c2*c3) >> 9]                                  (0..127)
  o1  = W1q[bucket] x0 + B1q ; skip = o1[L2-2] - o1[L2-1]
  x1  = clamp([(o1^2 + 20) >> 21, o1 >> 7], 0, 127)
  o2  = W2q[bucket] x1 + B2q ; x2 = clamp([(o2^2 + 5) >> 19, o2 >> 6], 0, 127)
  o3  = W3q[bucket] [x1, x2] + B3q
  pos = trunc(2*(o3 + skip) * 9600 / 32768)
  out = 2*pos + (psq_white - psq_black) * (+1 if white to move else -1)

in units of 1/19200 of the float model output.  The +20 / +5 are
floor(1e-5 * 2^21) / floor(1e-5 * 2^19): the images of the 1e-5 that
model/quantize.py:41 adds before its floor.  Shifts are arithmetic (floor).
"""

from __future__ import annotations

import numpy as np


DEFAULT_SCALES = {"ft": 256.0, "psqt": 9600.0, "l1": 128.0, "l2": 64.0, "out": 128.0, "hidden": 128.0}


def quantize_params(params: dict, L1: int, scales: dict = DEFAULT_SCALES) -> dict:
    """Round float parameters (numpy arrays, layout of oracle.model_oracle) onto
    the integer grids of model/quantize.py:100-110 (weights at their layer
    scale, biases at layer scale x hidden scale).  np.rint rounds half to even
    like torch.round."""
    count = params["out_w"].shape[0]
    w1 = params["l1_w"] + np.tile(params["l1f_w"], (count, 1))
    b1 = params["l1_b"] + np.tile(params["l1f_b"], count)
    h = scales["hidden"]
    r = lambda a, s: np.rint(np.asarray(a, dtype=np.float64) * s).astype(np.int64)  # noqa: E731
    return {
        "ft_w": r(params["ft_weight"][:, :L1], scales["ft"]),
        "ft_psqt": r(params["ft_weight"][:, L1:], scales["psqt"]),
        "ft_b": r(params["ft_bias"][:L1], scales["ft"]),
        "l1_w": r(w1, scales["l1"]), "l1_b": r(b1, scales["l1"] * h),
        "l2_w": r(params["l2_w"], scales["l2"]), "l2_b": r(params["l2_b"], scales["l2"] * h),
        "out_w": r(params["out_w"], scales["out"]), "out_b": r(params["out_b"], scales["out"] * h),
    }


def _accumulate(table, idx):
    """sum of table rows over the leading non-negative entries of each list."""
    B, K = idx.shape
    out = np.zeros((B, table.shape[1]), dtype=np.int64)
    alive = np.ones(B, dtype=bool)
    for k in range(K):
        alive &= idx[:, k] >= 0
        rows = np.where(alive, idx[:, k], 0)
        out += np.where(alive[:, None], table[rows], 0)
    return out


def integer_eval(qp: dict, white, black, stm_white, bucket, consts: dict) -> np.ndarray:
    """int64 [B]; `qp` from quantize_params, index lists int32 [B, K]."""
    L1 = qp["ft_w"].shape[1]
    h = L1 // 2
    count = qp["out_w"].shape[0]
    L2 = qp["l1_w"].shape[0] // count
    L3 = qp["l2_w"].shape[0] // count
    B = white.shape[0]
    stm = stm_white.astype(bool)

    acc_w = qp["ft_b"][None, :] + _accumulate(qp["ft_w"], white)
    acc_b = qp["ft_b"][None, :] + _accumulate(qp["ft_w"], black)
    psq_w = _accumulate(qp["ft_psqt"], white)[np.arange(B), bucket]
    psq_b = _accumulate(qp["ft_psqt"], black)[np.arange(B), bucket]
    first = np.where(stm[:, None], acc_w, acc_b)
    second = np.where(stm[:, None], acc_b, acc_w)
    c = np.clip(np.concatenate([first, second], axis=1), 0, consts["ft_max"])
    x0 = np.concatenate([(c[:, :h] * c[:, h:L1]) >> consts["ft_shift"],
                         (c[:, L1:L1 + h] * c[:, L1 + h:]) >> consts["ft_shift"]], axis=1)
    hm = consts["hidden_max"]

    w1 = qp["l1_w"].reshape(count, L2, L1)[bucket]
    o1 = np.einsum("boi,bi->bo", w1, x0) + qp["l1_b"].reshape(count, L2)[bucket]
    skip = (o1[:, L2 - 2] - o1[:, L2 - 1]) * consts["skip_mul"]
    x1 = np.clip(np.concatenate([(o1 * o1 + consts["sqr_eps_l1"]) >> consts["sqr_shift_l1"],
                                 o1 >> consts["lin_shift_l1"]], axis=1), 0, hm)
    w2 = qp["l2_w"].reshape(count, L3, 2 * L2)[bucket]
    o2 = np.einsum("boi,bi->bo", w2, x1) + qp["l2_b"].reshape(count, L3)[bucket]
    x2 = np.clip(np.concatenate([(o2 * o2 + consts["sqr_eps_l2"]) >> consts["sqr_shift_l2"],
                                 o2 >> consts["lin_shift_l2"]], axis=1), 0, hm)
    w3 = qp["out_w"][bucket]
    o3 = np.einsum("bi,bi->b", w3, np.concatenate([x1, x2], axis=1)) + qp["out_b"][bucket]
    num = 2 * (o3 + skip) * consts["out_mul"]
    pos = np.sign(num) * (np.abs(num) // consts["out_div"])
    return 2 * pos + (psq_w - psq_b) * np.where(stm, 1, -1)
