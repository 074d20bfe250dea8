"""`.nnue` file I/O.  CPU part: the writer's bytes are pinned to the reference
project's own serializer through SHA-256 digests of the file it wrote for the
same model (tests/golden/nnue_file.npz, made by tests/golden/make_golden.py),
for both storage forms; the LEB128 coder and the reader are checked by round
trips and on malformed input.  GPU part: the integer evaluation of the file's
tensors equals the reference's float64 fake-quantized forward."""

import hashlib
import io

import numpy as np
import pytest
import torch

from _util import load_golden, small_model_params, t


def _small_model():
    """This package's model with the weights make_golden.py put into the reference's."""
    from nnue_pytorch_b200.model import ModelConfig, NNUEModel

    p = small_model_params()
    m = NNUEModel("HalfKAv2_hm^", ModelConfig(L1=64, L2=32, L3=32))
    f32 = lambda a: torch.from_numpy(np.asarray(a)).float()  # noqa: E731
    with torch.no_grad():
        ft = m.input.features[0]
        ft.weight.copy_(f32(p["ft_real"]))
        ft.virtual_weight.copy_(f32(p["ft_virtual"]))
        m.input.bias.copy_(f32(p["ft_bias"]))
        ls = m.layer_stacks
        ls.l1.linear.weight.copy_(f32(p["l1_w"]))
        ls.l1.linear.bias.copy_(f32(p["l1_b"]))
        ls.l1.factorized_linear.weight.copy_(f32(p["l1f_w"]))
        ls.l1.factorized_linear.bias.copy_(f32(p["l1f_b"]))
        ls.l2.linear.weight.copy_(f32(p["l2_w"]))
        ls.l2.linear.bias.copy_(f32(p["l2_b"]))
        ls.output.linear.weight.copy_(f32(p["out_w"]))
        ls.output.linear.bias.copy_(f32(p["out_b"]))
    return m


def _scalar_leb128(v: int) -> bytes:
    out = []
    while True:
        byte = v & 0x7F
        v >>= 7
        if (v == 0 and not byte & 0x40) or (v == -1 and byte & 0x40):
            out.append(byte)
            return bytes(out)
        out.append(byte | 0x80)


@pytest.mark.parametrize("dtype,lo,hi", [(np.int8, -127, 127), (np.int16, -32767, 32767), (np.int32, -(2**31) + 1, 2**31 - 1)])
def test_leb128_round_trip_and_known_encodings(dtype, lo, hi):
    from nnue_pytorch_b200.serialize import decode_leb128, encode_leb128

    rng = np.random.default_rng(5)
    a = rng.integers(lo, hi, 20000).astype(dtype)
    a[:9] = [0, -1, 1, 63, 64, -64, -65, lo, hi]
    enc = encode_leb128(a)
    assert np.array_equal(decode_leb128(enc, a.size), a.astype(np.int64))
    assert enc[: sum(len(_scalar_leb128(int(x))) for x in a[:500])] == b"".join(_scalar_leb128(int(x)) for x in a[:500])
    assert encode_leb128(np.zeros(0, dtype=dtype)) == b"" and decode_leb128(b"", 0).size == 0
    assert encode_leb128(np.array([-128, 127, 128, 624485, -123456])) == bytes(
        [0x80, 0x7F, 0xFF, 0x00, 0x80, 0x01, 0xE5, 0x8E, 0x26, 0xC0, 0xBB, 0x78])
    with pytest.raises(EOFError):
        decode_leb128(enc, a.size + 1)


@pytest.mark.parametrize("compression", ["none", "leb128"])
def test_writer_bytes_equal_the_reference_serializer(compression):
    from nnue_pytorch_b200.serialize import to_bytes

    g = load_golden("nnue_file")
    data = to_bytes(_small_model(), ft_compression=compression)
    assert len(data) == int(g[f"length_{compression}"])
    assert data[:1024] == g[f"head_{compression}"].tobytes()
    assert data[-1024:] == g[f"tail_{compression}"].tobytes()
    assert hashlib.sha256(data).digest() == g[f"sha256_{compression}"].tobytes()


def test_reader_round_trip_and_errors():
    from nnue_pytorch_b200.model import ModelConfig
    from nnue_pytorch_b200.serialize import from_bytes, to_bytes

    m = _small_model()
    plain, packed = to_bytes(m), to_bytes(m, ft_compression="leb128")
    cfg = ModelConfig(L1=64, L2=32, L3=32)
    for data in (plain, packed):
        r = from_bytes(data, "HalfKAv2_hm^", cfg)
        assert to_bytes(r.model) == plain  # the factor layers are folded in, the integers are the same
        assert r.description.startswith("Network trained with")
        assert float(r.model.layer_stacks.l1.factorized_linear.weight.abs().sum()) == 0.0
    with pytest.raises(ValueError):  # another architecture's hash
        from_bytes(plain, "HalfKAv2_hm^", ModelConfig(L1=128, L2=32, L3=32))
    with pytest.raises(EOFError):
        from_bytes(plain[: len(plain) // 2], "HalfKAv2_hm^", cfg)
    with pytest.raises(ValueError):
        from_bytes(b"\0\0\0\0" + plain[4:], "HalfKAv2_hm^", cfg)
    with torch.no_grad():
        m.layer_stacks.l2.linear.weight[0, 0] = 5.0  # 5 * 64 does not fit int8
    with pytest.raises(RuntimeError, match="out of bounds"):
        to_bytes(m)


@pytest.mark.gpu
def test_integer_eval_of_the_file_matches_reference_float64():
    """Positions in the export layout (11 planes, real rows only) evaluated from
    the file's integers = the reference's float64 forward on the training layout."""
    from nnue_pytorch_b200 import positions
    from nnue_pytorch_b200.model import ModelConfig
    from nnue_pytorch_b200.serialize import load_quantized, to_bytes

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    dev = torch.device("cuda:0")
    g = load_golden("model_small")
    data = to_bytes(_small_model(), ft_compression="leb128")
    net = load_quantized(io.BytesIO(data), "HalfKAv2_hm^", ModelConfig(L1=64, L2=32, L3=32), dev)
    pos = positions.generate_positions(96, 21)
    lists = []
    for white_pov in (True, False):
        idx = positions.baseline_indices(pos, white_pov)
        idx[idx >= positions.NUM_REAL_BASELINE] = -1  # the exported net has no factor rows
        lists.append(t(np.ascontiguousarray(idx[:, :32])).to(dev))
    out = net.evaluate(lists[0], lists[1], t(pos.stm_white), t(pos.piece_count))
    assert np.array_equal(out.cpu().numpy().astype(np.int64), g["eval_int"][:, 0])
