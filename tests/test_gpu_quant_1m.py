"""BASELINE configs[4]: one million seeded positions through the integer
evaluation, compared for exact equality with the float64 fake-quantized forward
(the reference's definition of its quantized evaluation, restated in
oracle/model_oracle.py and run here on the GPU in float64 as the checker).
Architecture of configs[1]: 23232 -> 3072, eight buckets, L2 = L3 = 32."""

import time

import numpy as np
import pytest
import torch

from _util import t

pytestmark = pytest.mark.gpu

CHUNK = 16384
N_CHUNKS = 62  # 62 * 16384 = 1 015 808 positions


def test_one_million_positions_bit_exact():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from oracle import model_oracle
    from nnue_pytorch_b200 import positions
    from nnue_pytorch_b200.quantized_eval import QuantizedNet
    from test_gpu_quant_and_model import _random_quant_params

    dev = torch.device("cuda:0")
    L1 = 3072
    p = _random_quant_params(L1, positions.NUM_INPUTS_BASELINE, np.random.default_rng(4))
    p64 = {k: t(np.asarray(v), torch.float64).to(dev) for k, v in p.items()}
    l1_w = p64["l1_w"] + p64["l1f_w"].repeat(8, 1)
    l1_b = p64["l1_b"] + p64["l1f_b"].repeat(8)
    net = QuantizedNet(p64["ft_weight"], p64["ft_bias"], l1_w, l1_b, p64["l2_w"], p64["l2_b"], p64["out_w"],
                       p64["out_b"], L1, 8)
    total = mismatches = 0
    gpu_ms = 0.0
    distinct = set()
    for c in range(N_CHUNKS):
        b = positions.generate_batch(CHUNK, 10_000 + c, layout="baseline")
        us, them, white, black = (t(x).to(dev) for x in (b.us, b.them, b.white, b.black))
        pc = t(b.piece_count).to(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        got = net.evaluate(white, black, us[:, 0] > 0.5, pc)
        e1.record()
        want = torch.round(model_oracle.forward(p64, us.double(), them.double(), white, black, pc) * 19200)
        torch.cuda.synchronize()
        gpu_ms += e0.elapsed_time(e1)
        mismatches += int((got.to(torch.int64) != want[:, 0].to(torch.int64)).sum())
        total += CHUNK
        if c < 4:
            distinct.update(got[:2048].tolist())
    assert total >= 1_000_000
    assert mismatches == 0, f"{mismatches} of {total} integer evaluations differ"
    assert len(distinct) > 2000  # the net is not degenerate
    print(f"\nquantized eval: {total} positions, {total / (gpu_ms * 1e-3):.3e} positions/s on the GPU")
    _ = time
