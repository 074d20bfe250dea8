"""Index lists of the reference's default feature set
`Full_Threats+PP_3Wide+HalfKAv2_hm^` (88944 table rows, up to 288 active
indices per perspective), built on the host from board positions.

Restates the extractors of the reference's loader,
data_loader/cpp/training_data_loader.cpp of the reference project:
  :20-73    HalfKAv2_hm   one index per piece: oriented square + plane * 64 + king bucket * 768
  :85-302   Full_Threats  one index per (attacker, from, target, to) pair, pawns never target pawns,
                          kings neither attack nor are attacked, same-type pairs counted once
  :306-388  PP_3Wide      one index per pair of pawns on the same or adjacent files
  :394-430  composition   lists concatenated in that order, each block's indices shifted by the
                          sizes of the blocks before it
in the order the loader emits them (own colour first, squares ascending), so the lists can be
compared entry for entry.  A board is a sequence of 64 piece codes, a1 = 0 ... h8 = 63:
0 = empty, else 1 + 2 * type + is_black with type 0..5 = pawn, knight, bishop, rook, queen, king.

Plain Python over small tables: meant for tests, fixtures and benchmark inputs, not for a
training loader.
"""

from __future__ import annotations

import numpy as np

from .positions import KING_BUCKETS, PositionBatch

PAWN, KNIGHT, BISHOP, ROOK, QUEEN, KING = range(6)
THREAT_INPUTS = 59808
PAWN_PAIR_INPUTS = 96 * 95 // 2          # 4560
HALFKA_INPUTS = 768 * 32                 # 24576
FULL_INPUTS = THREAT_INPUTS + PAWN_PAIR_INPUTS + HALFKA_INPUTS   # 88944
THREAT_MAX_ACTIVE = PAWN_PAIR_MAX_ACTIVE = 128
FULL_MAX_ACTIVE = THREAT_MAX_ACTIVE + PAWN_PAIR_MAX_ACTIVE + 32  # 288

_NUM_VALID_TARGETS = (4, 10, 8, 8, 10, 0)
# target slot by (attacker type, attacked type); -1 = pair not represented
_SLOT = (
    (-1, 0, -1, 1, -1, -1),
    (0, 1, 2, 3, 4, -1),
    (0, 1, 2, 3, -1, -1),
    (0, 1, 2, 3, -1, -1),
    (0, 1, 2, 3, 4, -1),
    (-1, -1, -1, -1, -1, -1),
)


def _leaper(sq: int, deltas) -> int:
    f, r = sq & 7, sq >> 3
    m = 0
    for df, dr in deltas:
        ff, rr = f + df, r + dr
        if 0 <= ff < 8 and 0 <= rr < 8:
            m |= 1 << (rr * 8 + ff)
    return m


def _ray_attacks(sq: int, dirs, occupied: int) -> int:
    f, r = sq & 7, sq >> 3
    m = 0
    for df, dr in dirs:
        ff, rr = f + df, r + dr
        while 0 <= ff < 8 and 0 <= rr < 8:
            bit = 1 << (rr * 8 + ff)
            m |= bit
            if occupied & bit:
                break
            ff, rr = ff + df, rr + dr
    return m


_DIAG = ((1, 1), (1, -1), (-1, 1), (-1, -1))
_ORTH = ((1, 0), (-1, 0), (0, 1), (0, -1))
_KNIGHT_D = ((1, 2), (2, 1), (2, -1), (1, -2), (-1, -2), (-2, -1), (-2, 1), (-1, 2))


def _pawn_attacks(sq: int, black: bool) -> int:
    return _leaper(sq, ((1, -1), (-1, -1)) if black else ((1, 1), (-1, 1)))


# attacks on an empty board, by piece type (pawns by colour)
_PSEUDO = {
    KNIGHT: [_leaper(s, _KNIGHT_D) for s in range(64)],
    BISHOP: [_ray_attacks(s, _DIAG, 0) for s in range(64)],
    ROOK: [_ray_attacks(s, _ORTH, 0) for s in range(64)],
    QUEEN: [_ray_attacks(s, _DIAG + _ORTH, 0) for s in range(64)],
}
_PAWN_ATT = [[_pawn_attacks(s, False) for s in range(64)], [_pawn_attacks(s, True) for s in range(64)]]


def _threat_offsets():
    """Per attacker (colour * 5 + type, kings excluded): offset of each from-square inside the attacker's
    block ([0..63]), attacks per target slot ([64]) and first index of the attacker's block ([65])."""
    table, piece_offset = [], 0
    for piece in range(10):
        black, ptype = piece >= 5, piece % 5
        row, square_offset = [0] * 66, 0
        for frm in range(64):
            row[frm] = square_offset
            if ptype == PAWN:
                if 8 <= frm <= 55:
                    square_offset += bin(_PAWN_ATT[black][frm]).count("1")
            else:
                square_offset += bin(_PSEUDO[ptype][frm]).count("1")
        row[64], row[65] = square_offset, piece_offset
        piece_offset += _NUM_VALID_TARGETS[ptype] * square_offset
        table.append(row)
    assert piece_offset == THREAT_INPUTS
    return table


_OFFSETS = _threat_offsets()


def _orient(white_pov: bool, ksq: int) -> int:
    """XOR mask that puts the perspective's king on files a-d and, for black, flips the ranks."""
    return (7 if (ksq & 7) >= 4 else 0) ^ (0 if white_pov else 56)


def _bits(m: int):
    while m:
        low = m & -m
        yield low.bit_length() - 1
        m ^= low


def _decode(code: int):
    """(type 0..5, is_black) of a non-empty board code."""
    return (code - 1) >> 1, bool((code - 1) & 1)


def threat_index(white_pov: bool, a_type: int, a_black: bool, frm: int, to: int, d_type: int, d_black: bool, ksq: int) -> int:
    o = _orient(white_pov, ksq)
    frm, to = frm ^ o, to ^ o
    if not white_pov:
        a_black, d_black = not a_black, not d_black
    slot = _SLOT[a_type][d_type]
    if slot < 0:
        return -1
    enemy = a_black != d_black
    if a_type == d_type and (enemy or a_type != PAWN) and frm < to:
        return -1
    attacks = _PAWN_ATT[a_black][frm] if a_type == PAWN else _PSEUDO[a_type][frm]
    off = _OFFSETS[int(a_black) * 5 + a_type]
    below = bin(((1 << to) - 1) & attacks).count("1")
    return off[65] + (int(d_black) * (_NUM_VALID_TARGETS[a_type] // 2) + slot) * off[64] + off[frm] + below


def threat_features(board, white_pov: bool) -> list[int]:
    occ = pawns = kings = 0
    by_piece: dict[tuple[int, bool], int] = {}
    for sq, code in enumerate(board):
        if code:
            t, blk = _decode(code)
            bit = 1 << sq
            occ |= bit
            by_piece[(t, blk)] = by_piece.get((t, blk), 0) | bit
            if t == PAWN:
                pawns |= bit
            elif t == KING:
                kings |= bit
    ksq = (by_piece[(KING, not white_pov)].bit_length() - 1)
    no_kings = occ & ~kings
    out = []
    for black in ((False, True) if white_pov else (True, False)):   # own colour first
        bb = by_piece.get((PAWN, black), 0)
        diag_targets = no_kings & ~pawns                              # pawn pairs belong to PP_3Wide
        not_a, not_h = 0xFEFEFEFEFEFEFEFE, 0x7F7F7F7F7F7F7F7F
        full = (1 << 64) - 1
        if not black:
            right, r_delta = ((bb & not_h) << 9) & full, 9            # towards the h-file and up
            left, l_delta = ((bb & not_a) << 7) & full, 7
        else:
            right, r_delta = (bb & not_a) >> 9, -9                    # towards the a-file and down
            left, l_delta = (bb & not_h) >> 7, -7
        for shifted, delta in ((right, r_delta), (left, l_delta)):
            for to in _bits(shifted & diag_targets):
                d_type, d_black = _decode(board[to])
                idx = threat_index(white_pov, PAWN, black, to - delta, to, d_type, d_black, ksq)
                if idx >= 0:
                    out.append(idx)
        for a_type in (KNIGHT, BISHOP, ROOK, QUEEN):
            for frm in _bits(by_piece.get((a_type, black), 0)):
                if a_type == KNIGHT:
                    att = _PSEUDO[KNIGHT][frm]
                else:
                    dirs = _DIAG if a_type == BISHOP else _ORTH if a_type == ROOK else _DIAG + _ORTH
                    att = _ray_attacks(frm, dirs, occ)
                for to in _bits(att & no_kings):
                    d_type, d_black = _decode(board[to])
                    idx = threat_index(white_pov, a_type, black, frm, to, d_type, d_black, ksq)
                    if idx >= 0:
                        out.append(idx)
    return out


_FILE_A = 0x0101010101010101


def _pawn_pair_mask(sq: int) -> int:
    f = sq & 7
    files = _FILE_A << f
    if f > 0:
        files |= _FILE_A << (f - 1)
    if f < 7:
        files |= _FILE_A << (f + 1)
    return files & ~0xFF & ~(0xFF << 56) & ~(1 << sq) & ((1 << 64) - 1)


def pawn_pair_features(board, white_pov: bool) -> list[int]:
    pawns = {False: 0, True: 0}
    ksq = -1
    for sq, code in enumerate(board):
        if code:
            t, blk = _decode(code)
            if t == PAWN:
                pawns[blk] |= 1 << sq
            elif t == KING and blk == (not white_pov):
                ksq = sq
    all_pawns = pawns[False] | pawns[True]
    o = _orient(white_pov, ksq)
    out = []
    for black in ((False, True) if white_pov else (True, False)):
        for frm in _bits(pawns[black]):
            for to in _bits(_pawn_pair_mask(frm) & all_pawns):
                if frm < to:
                    continue
                other_black = bool(pawns[True] >> to & 1)
                fo, to_o = frm ^ o, to ^ o
                if not (8 <= fo <= 55 and 8 <= to_o <= 55):
                    continue
                ca, cb = int(black) ^ int(not white_pov), int(other_black) ^ int(not white_pov)
                id_a, id_b = 48 * ca + fo - 8, 48 * cb + to_o - 8
                hi, lo = max(id_a, id_b), min(id_a, id_b)
                out.append(hi * (hi - 1) // 2 + lo)
    return out


def halfka_features(board, white_pov: bool) -> list[int]:
    """Native 12-plane HalfKAv2_hm indices in square order (model/modules/features/halfka_v2_hm.py:27-36)."""
    ksq = next(sq for sq, code in enumerate(board) if code and _decode(code) == (KING, not white_pov))
    flip = (7 if (ksq & 7) < 4 else 0) ^ (0 if white_pov else 56)
    bucket = int(KING_BUCKETS[ksq ^ flip])
    out = []
    for sq, code in enumerate(board):
        if code:
            t, blk = _decode(code)
            theirs = blk == white_pov   # white perspective: black pieces are "theirs"
            out.append((sq ^ flip) + (t * 2 + int(theirs)) * 64 + bucket * 768)
    return out


def composed_features(board, white_pov: bool) -> list[int]:
    """`Full_Threats+PP_3Wide+HalfKAv2_hm^`: the three lists back to back with the blocks' row offsets."""
    return (threat_features(board, white_pov)
            + [THREAT_INPUTS + i for i in pawn_pair_features(board, white_pov)]
            + [THREAT_INPUTS + PAWN_PAIR_INPUTS + i for i in halfka_features(board, white_pov)])


def boards_of(pos: PositionBatch) -> np.ndarray:
    """[B, 64] board codes of generated positions.  A pawn the generator put on the first or last rank
    becomes a knight: the threat tables have no rows for such pawns."""
    B = pos.squares.shape[0]
    boards = np.zeros((B, 64), dtype=np.int8)
    live = np.arange(32)[None, :] < pos.piece_count[:, None]
    ptype = pos.piece_type - 1
    rank = pos.squares >> 3
    ptype = np.where((ptype == PAWN) & ((rank == 0) | (rank == 7)), KNIGHT, ptype)
    code = 1 + 2 * ptype + (~pos.is_white).astype(np.int64)
    rows = np.repeat(np.arange(B), 32).reshape(B, 32)
    boards[rows[live], pos.squares[live]] = code[live]
    return boards


def full_feature_lists(boards, max_active: int = FULL_MAX_ACTIVE) -> tuple[np.ndarray, np.ndarray]:
    """(white, black) int32 [B, max_active] lists of the composed feature set, -1 padded."""
    B = len(boards)
    out = [np.full((B, max_active), -1, dtype=np.int32) for _ in range(2)]
    for b in range(B):
        board = [int(x) for x in boards[b]]
        for side, white_pov in enumerate((True, False)):
            lst = composed_features(board, white_pov)
            if len(lst) > max_active:
                raise ValueError(f"position {b}: {len(lst)} active features exceed {max_active}")
            out[side][b, : len(lst)] = lst
    return out[0], out[1]
