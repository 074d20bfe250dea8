"""The default feature set `Full_Threats+PP_3Wide+HalfKAv2_hm^`: index lists and feature blocks.

The host index builder (nnue_pytorch_b200/full_features.py) is pinned entry for entry against
tests/golden/full_features.npz: 300 real positions from the reference project's sample binpack
run through the reference loader's own extractors (tests/golden/make_golden.py compiles them
from the reference sources)."""

import numpy as np
import torch

from _util import load_golden


def test_index_lists_equal_the_reference_extractors_on_real_positions():
    from nnue_pytorch_b200 import full_features as ff

    g = load_golden("full_features")
    boards = g["boards"]
    assert boards.shape == (300, 64)
    builders = {"halfka": ff.halfka_features, "threats": ff.threat_features, "pawn_pairs": ff.pawn_pair_features}
    longest = dict.fromkeys(builders, 0)
    for i in range(boards.shape[0]):
        board = [int(x) for x in boards[i]]
        for side, white_pov in enumerate((True, False)):
            for name, fn in builders.items():
                want = g[name][i, side]
                want = want[want >= 0].tolist()
                assert fn(board, white_pov) == want, (i, side, name)
                longest[name] = max(longest[name], len(want))
            whole = ff.composed_features(board, white_pov)
            assert len(whole) <= ff.FULL_MAX_ACTIVE and max(whole) < ff.FULL_INPUTS and min(whole) >= 0
    assert longest["threats"] > 30 and longest["pawn_pairs"] > 20 and longest["halfka"] == 32


def test_threat_table_size_and_block_offsets():
    from nnue_pytorch_b200 import full_features as ff

    assert ff.FULL_INPUTS == 88944 and ff.FULL_MAX_ACTIVE == 288
    # the start position: every list has its block's indices inside the block's row range
    back = [3, 1, 2, 4, 5, 2, 1, 3]
    board = [0] * 64
    for f, t in enumerate(back):
        board[f], board[56 + f] = 1 + 2 * t, 2 + 2 * t
        board[8 + f], board[48 + f] = 1, 2
    for white_pov in (True, False):
        lst = ff.composed_features(board, white_pov)
        thr = [i for i in lst if i < ff.THREAT_INPUTS]
        pp = [i for i in lst if ff.THREAT_INPUTS <= i < ff.THREAT_INPUTS + ff.PAWN_PAIR_INPUTS]
        hk = [i for i in lst if i >= ff.THREAT_INPUTS + ff.PAWN_PAIR_INPUTS]
        assert len(hk) == 32 and len(pp) == 36 and len(thr) == 28
        assert lst == thr + pp + hk  # blocks in order
    # the start position is its own mirror image: both perspectives see the same features (the order inside a
    # list follows the squares of the unmirrored board, so it differs)
    assert sorted(ff.composed_features(board, True)) == sorted(ff.composed_features(board, False))


def test_generated_positions_give_valid_lists():
    from nnue_pytorch_b200 import full_features as ff, positions

    pos = positions.generate_positions(64, 3)
    boards = ff.boards_of(pos)
    assert ((boards > 0).sum(axis=1) == pos.piece_count).all()
    rank = np.arange(64) // 8
    assert not (((boards == 1) | (boards == 2)) & ((rank == 0) | (rank == 7))[None, :]).any()  # no pawn on rank 1 / 8
    white, black = ff.full_feature_lists(boards)
    assert white.shape == (64, 288) and white.dtype == np.int32
    for lists in (white, black):
        n = (lists >= 0).sum(axis=1)
        assert (n >= pos.piece_count).all()
        assert ((lists >= 0).cumsum(axis=1)[np.arange(64), np.maximum(n - 1, 0)] == n).all()  # padding on the right only
        assert lists.max() < ff.FULL_INPUTS


def test_default_feature_set_blocks():
    from nnue_pytorch_b200.features import DEFAULT_FEATURES, get_feature_cls
    from nnue_pytorch_b200.quantize import QuantizationManager

    classes = get_feature_cls(DEFAULT_FEATURES)
    blocks = [c(72) for c in classes]
    assert [b.NUM_INPUTS for b in blocks] == [59808, 4560, 24576]
    assert sum(b.MAX_ACTIVE_FEATURES for b in blocks) == 288
    q = QuantizationManager()
    with torch.no_grad():
        blocks[0].weight[5, 3] = 3.0
        blocks[0].weight[6, 3] = -3.0
    blocks[0].clip_weights(q)
    assert float(blocks[0].weight.max()) == 127 / 256 and float(blocks[0].weight.min()) == -127 / 256
    blocks[0].init_weights(8, 600.0)
    assert float(blocks[0].weight[:, 64:].abs().max()) == 0.0
    assert blocks[0].EXPORT_WEIGHT_DTYPE == torch.int8 and blocks[2].EXPORT_WEIGHT_DTYPE == torch.int16
