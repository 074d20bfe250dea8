"""`FusedLayerStackFunction`: the bucketed layer stack as one autograd op.

Same mathematics as `LayerStacks.forward` of the reference project
(model/modules/layer_stacks.py:33-84 with model/modules/stacked_linear.py:38-66):
three bucketed linear layers, squared + linear clipped activations with
straight-through fake quantization, the skip connection from the first
layer's last two outputs and the output fake quantization.  The reference
multiplies every position with the weights of all buckets and then selects;
the kernels behind this op (csrc/layer_stack*.cu) group the batch by bucket
and multiply each position with its own bucket's block only.

Inputs are the effective weights of this step (factor already merged, weight
fake quantization already applied by the caller, where gradients flow through
ordinary autograd): W1 [C*32, L1], b1 [C*32], W2 [C*32, 64], b2 [C*32],
W3 [C, 128], b3 [C].
"""

from __future__ import annotations

import ctypes as C

import torch
from torch import autograd

from . import _lib
from ._launch import _ptr, _require_cuda, _span, _stream


def _params(quantization, fake_quantize_acts: bool) -> _lib.LsParams:
    c = quantization.config
    p = _lib.LsParams()
    p.act_scale = float(c.hidden_quantized_one) if fake_quantize_acts else 0.0
    p.act_eps = 1e-5
    p.sqr_corr = float(quantization.sqr_crelu_correction_factor)
    p.max_hidden = float(quantization.max_hidden_activation)
    p.out_den = float(int(c.hidden_quantized_one * c.weight_scale_l_out * 2.0))
    p.out_mul = float(int(c.nnue2score * c.weight_scale_out))
    p.quantize_out = 1 if fake_quantize_acts else 0
    return p


def supported(x: torch.Tensor, l1: int, l2: int, l3: int, count: int) -> bool:
    return x.is_cuda and x.dtype == torch.float32 and l2 == 32 and l3 == 32 and l1 % 32 == 0 and 1 <= count <= 16


_PLAN_STREAMS: dict[int, torch.cuda.Stream] = {}


class PlanAhead:
    """The bucket plan of a batch, built on a second stream.  It depends on
    the bucket indices only, so a caller that knows them early (before the
    feature transformer runs) gets the plan for free, beside that work."""

    def __init__(self, bucket: torch.Tensor, count: int):
        dev = _require_cuda(bucket)
        key = dev.index if dev.index is not None else torch.cuda.current_device()
        side = _PLAN_STREAMS.get(key)
        if side is None:
            side = _PLAN_STREAMS[key] = torch.cuda.Stream(dev)
        lib = _lib.load()
        self.bucket = bucket.reshape(-1).to(torch.int64).contiguous()
        self.count, self.B = int(count), self.bucket.numel()
        self.plan = torch.empty(lib.nnue_ls_plan_bytes(self.B, count) // 4 + 4, dtype=torch.int32, device=dev)
        cur = torch.cuda.current_stream(dev)
        side.wait_stream(cur)  # the bucket indices (and the plan's memory) are ready on the caller's stream
        with torch.cuda.device(dev):
            _lib.check(lib.nnue_ls_plan(_ptr(self.bucket), self.B, count, _ptr(self.plan), self.plan.numel() * 4,
                                        side.cuda_stream), "nnue_ls_plan")
        self.bucket.record_stream(side)
        self.plan.record_stream(side)
        self.ready = torch.cuda.Event()
        self.ready.record(side)

    def take(self, dev, B: int, count: int) -> torch.Tensor:
        assert self.B == B and self.count == count, "the plan was built for another batch"
        torch.cuda.current_stream(dev).wait_event(self.ready)
        return self.plan


# False: the first layer's input gradient stays on the fp32 FMA kernel also in the quantized model
TENSOR_CORE_DX = True


class FusedLayerStackFunction(autograd.Function):
    @staticmethod
    def forward(ctx, x, bucket, W1, b1, W2, b2, W3, b3, quantization, fake_quantize_acts, plan_ahead=None,
                exact_tf32=False):
        """`exact_tf32`: x and W1 are exactly representable in TF32 (the quantized model: activations on the
        1/128 grid, fake-quantized weights); the first layer then runs on the tensor cores, same bits."""
        dev = _require_cuda(x, bucket, W1, b1, W2, b2, W3, b3)
        x, W1, b1, W2, b2, W3, b3 = (t.contiguous() for t in (x, W1, b1, W2, b2, W3, b3))
        bucket = bucket.reshape(-1).to(torch.int64).contiguous()
        B, L1 = x.shape
        count = W3.shape[0]
        assert W1.shape == (count * 32, L1) and W2.shape == (count * 32, 64) and W3.shape == (count, 128)
        lib = _lib.load()
        params = _params(quantization, fake_quantize_acts)
        if plan_ahead is not None:
            plan = plan_ahead.take(dev, B, count)
        else:
            plan = torch.empty(lib.nnue_ls_plan_bytes(B, count) // 4 + 4, dtype=torch.int32, device=dev)
        o1 = torch.empty(B, 32, device=dev)
        o2 = torch.empty(B, 32, device=dev)
        y = torch.empty(B, 1, device=dev)
        s = _stream(dev)
        with torch.cuda.device(dev), _span("layer_stack_fwd", dev):
            if plan_ahead is None:
                _lib.check(lib.nnue_ls_plan(_ptr(bucket), B, count, _ptr(plan), plan.numel() * 4, s), "nnue_ls_plan")
            with _span("ls_l1_fwd", dev):
                l1_fwd = lib.nnue_ls_l1_fwd_tc if exact_tf32 else lib.nnue_ls_l1_fwd
                _lib.check(l1_fwd(_ptr(x), _ptr(W1), _ptr(b1), _ptr(plan), _ptr(o1), B, L1, count, s), "nnue_ls_l1_fwd")
            _lib.check(lib.nnue_ls_tail_fwd(_ptr(o1), _ptr(plan), _ptr(W2), _ptr(b2), _ptr(W3), _ptr(b3.reshape(-1)),
                                            C.byref(params), _ptr(o2), _ptr(y), B, count, s), "nnue_ls_tail_fwd")
        ctx.save_for_backward(x, W1, W2, W3, o1, o2, plan)
        ctx.params, ctx.count, ctx.b3_shape = params, count, tuple(b3.shape)
        ctx.exact_tf32 = bool(exact_tf32)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, W1, W2, W3, o1, o2, plan = ctx.saved_tensors
        dev = x.device
        B, L1 = x.shape
        count = ctx.count
        lib = _lib.load()
        gy = gy.contiguous()
        d_o1 = torch.empty(B, 32, device=dev)
        dW1 = torch.empty_like(W1)
        db1 = torch.empty(count * 32, device=dev)
        dW2 = torch.empty_like(W2)
        db2 = torch.empty(count * 32, device=dev)
        dW3 = torch.empty_like(W3)
        db3 = torch.empty(count, device=dev)
        dx = torch.empty_like(x) if ctx.needs_input_grad[0] else None
        ws = torch.empty(lib.nnue_ls_tail_bwd_workspace_bytes(B, count), dtype=torch.uint8, device=dev)
        s = _stream(dev)
        with torch.cuda.device(dev), _span("layer_stack_bwd", dev):
            _lib.check(lib.nnue_ls_tail_bwd(_ptr(o1), _ptr(o2), _ptr(plan), _ptr(W2), _ptr(W3), _ptr(gy),
                                            C.byref(ctx.params), _ptr(d_o1), _ptr(dW2), _ptr(db2), _ptr(dW3),
                                            _ptr(db3), _ptr(ws), ws.numel(), B, count, s), "nnue_ls_tail_bwd")
            with _span("ls_l1_bwd", dev):
                if ctx.exact_tf32 and dx is not None and L1 % 128 == 0 and TENSOR_CORE_DX:
                    # W1 is exact in TF32 (see forward): the input gradient on the tensor cores
                    ws1 = torch.empty(lib.nnue_ls_l1_bwd_tc_workspace_bytes(L1, count), dtype=torch.uint8, device=dev)
                    _lib.check(lib.nnue_ls_l1_bwd_tc(_ptr(x), _ptr(W1), _ptr(d_o1), _ptr(plan), _ptr(dx), _ptr(dW1),
                                                     _ptr(db1), B, L1, count, _ptr(ws1), ws1.numel(), s), "nnue_ls_l1_bwd_tc")
                else:
                    _lib.check(lib.nnue_ls_l1_bwd(_ptr(x), _ptr(W1), _ptr(d_o1), _ptr(plan), _ptr(dx), _ptr(dW1),
                                                  _ptr(db1), B, L1, count, s), "nnue_ls_l1_bwd")
        return dx, None, dW1, db1, dW2, db2, dW3, db3.view(ctx.b3_shape), None, None, None, None


class LayerStackWeightsFunction(autograd.Function):
    """(w1, b1, w2, b2, w3, b3) = effective weights of this step: the shared
    factor layer merged into every bucket of the first layer
    (model/modules/stacked_linear.py:96-127 of the reference project) and the
    weight fake quantization with its straight-through gradient
    (model/quantize.py:49-50), written by one kernel launch.  Backward: every
    gradient passes through; the factor layer receives the first layer's
    gradient summed over buckets."""

    @staticmethod
    def forward(ctx, l1_w, l1_b, l1f_w, l1f_b, l2_w, l2_b, out_w, out_b, quantization, fake_quantize_weights):
        dev = _require_cuda(l1_w, l1_b, l1f_w, l1f_b, l2_w, l2_b, out_w, out_b)
        ins = [t.detach().contiguous() for t in (l1_w, l1_b, l1f_w, l1f_b, l2_w, l2_b, out_w, out_b)]
        count = out_w.shape[0]
        L1 = l1_w.shape[1]
        assert l1_w.shape == (count * 32, L1) and l1f_w.shape == (32, L1) and l2_w.shape == (count * 32, 64)
        assert out_w.shape == (count, 128) and l1_b.numel() == count * 32 and l1f_b.numel() == 32
        sc = _lib.LsWeightScales()
        d = quantization.weight_scales_dict
        sc.w1, sc.b1 = d["ls_l1_weight"], d["ls_l1_bias"]
        sc.w2, sc.b2 = d["ls_l2_weight"], d["ls_l2_bias"]
        sc.w3, sc.b3 = d["ls_output_weight"], d["ls_output_bias"]
        sc.quantize = 1 if fake_quantize_weights else 0
        outs = [torch.empty_like(ins[i]) for i in (0, 1, 4, 5, 6, 7)]
        with torch.cuda.device(dev):
            _lib.check(
                _lib.load().nnue_ls_effective_weights(*[_ptr(t) for t in ins], C.byref(sc), *[_ptr(t) for t in outs],
                                                      L1, count, _stream(dev)),
                "nnue_ls_effective_weights",
            )
        ctx.dims = (L1, count, l1f_b.shape)
        return tuple(outs)

    @staticmethod
    def backward(ctx, g_w1, g_b1, g_w2, g_b2, g_w3, g_b3):
        L1, count, fb_shape = ctx.dims
        g_w1, g_b1 = g_w1.contiguous(), g_b1.contiguous()
        dev = g_w1.device
        g_fw = torch.empty(32, L1, device=dev)
        g_fb = torch.empty(fb_shape, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().nnue_ls_fold_grads(_ptr(g_w1), _ptr(g_b1), _ptr(g_fw), _ptr(g_fb), L1, count,
                                                      _stream(dev)), "nnue_ls_fold_grads")
        return g_w1, g_b1, g_fw, g_fb, g_w2, g_b2, g_w3, g_b3, None, None
