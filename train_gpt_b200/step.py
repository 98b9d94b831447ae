"""The caller of the hot path: one GPT pre-training step with the FP8 linears and the fused
norm, data-parallel over the GPUs of a node.

This is the restatement of train-gpt's step that the benchmark needs (model.py:57-98 as
re-built by bench_fp8_norm.py:81-128, losses.py:8-12, train.py:114-137), not a model zoo:
attention (torch SDPA), embedding, loss and AdamW are torch glue; the six projections per
layer and the norms run on this package's kernels through the reference's `mm` / `norm` seam.

    mm   "fp8"      block_scaled_matmul, 128x128 weight tiles, FP8 dgrad + wgrad
         "fp8_ref"  block_scaled_matmul exactly as the reference calls it (128x1 tiles, bf16 STE backward)
         "bf16"     a @ b (bench_fp8_norm.py:130)
    norm "fused"    rms_norm_quant feeding q/k/v (and up) from ONE quantised activation (FP8 mm only)
         "kernel"   kernels.rms_norm;  "pure": kernels._rms_norm_pure
         "torch_reference"  kernels.py:30-33 written with torch ops: the comparator the loss-curve
                    parity test and the CPU (gloo) tests of the gradient exchange run against

Differences from model.py that the benchmark's training configuration asks for are switches: GELU
(default there) or the reference's squared ReLU (model.py:72); learned positions, separate
q/k/v, untied head, tanh logit cap 15 and the 0.02 / 0.02/sqrt(2L) init follow model.py.
No per-block rematerialisation (the reference's `use_remat` trades compute for memory; 180 GB
does not need it at these sizes).
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import fp8, kernels, losses, ops, optim
from .dp import GradBuckets


@dataclass(frozen=True)
class StepConfig:
    vocab_size: int = 50304
    seq_len: int = 1024
    d_model: int = 1024
    n_layers: int = 24
    n_heads: int = 16
    head_dim: int = 64
    d_ff: int = 4096
    init_std: float = 0.02          # config.py:16
    rms_eps: float = 1e-5           # config.py:17
    logit_cap: float = 15.0         # config.py:19
    activation: str = "gelu"        # "gelu" (the benchmark's training configuration) or "relu2" (model.py:72)
    mm: str = "fp8"
    mlp: str = "fused"              # "fused": activation and its gradient folded into the quantisers (FP8 mm only); "unfused"
    norm: str = "fused"
    qkv: str = "fused"              # "fused": one dgrad GEMM contracts over the gradients of q, k and v (FP8 mm, norm "fused"); "separate"
    residual: str = "fused"         # "fused": the residual add runs inside the norm after it, its gradient fan-in inside that
                                    # norm's backward (norm "fused", FP8 mm, d_model <= 2048); "separate": elementwise adds
    loss: str = "fused"             # "fused": one CUDA pass each way over the logits; "torch": op by op (CPU tests)
    optimizer: str = "fused"        # "fused": optim.ClippedAdamW (CUDA kernels); "torch": torch.optim.AdamW + tensor-op clip
    flat_parameters: bool = True    # optimizer "fused": a bucket's parameters and moments are slices of flat tensors, one AdamW launch per bucket
    defer_exchange: bool = True     # more than one rank: a finished bucket's all-reduce is launched just before the next attention backward, not at once
    direct_grads: bool = True       # mm "fp8": weight-gradient GEMMs write into the gradient buckets (dp.GradSlot) instead of autograd adding into zeroed ones
    lr: float = 3e-4
    weight_decay: float = 0.1       # train.py make_optimizer default use
    clip_norm: float = 1.0


# SMs kept free of GEMM thread blocks while gradients are exchanged.  Measured on 2 GPUs (ms per step, graph replay):
# 0 -> 99.4, 8 -> 101.6, 16 -> 101.7, 32 -> 103.8: the all-reduce kernels themselves shrink (6.3 -> 2.8 ms summed over a
# step) but they were hidden behind the backward pass anyway, and the GEMMs lose more than that.  So: none.
RESERVED_SMS_DP = 0

SMALL = dict(vocab_size=256, seq_len=128, d_model=128, n_layers=2, n_heads=4, head_dim=32, d_ff=512)  # config.py:32-40


class _NormQuant(torch.autograd.Function):
    """rms_norm whose forward also emits the 1x128-quantised form of its output; the bf16
    output carries the gradient, the quantised pair rides along for the GEMMs."""

    @staticmethod
    def forward(ctx, x, gamma, eps):
        q, s, y, _ = ops.rmsnorm_quant_fwd(x, gamma, eps, want_y=True)
        ctx.save_for_backward(x, gamma)
        ctx.eps = eps
        ctx.mark_non_differentiable(q, s)
        ctx.set_materialize_grads(False)        # no zero-filled "gradients" for the quantised pair
        return y, q, s

    @staticmethod
    def backward(ctx, gy, _gq, _gs):
        x, gamma = ctx.saved_tensors
        if gy is None:
            return None, None, None
        dx, dgamma = ops.rmsnorm_bwd(x, gamma, gy.contiguous(), ctx.eps)
        return dx, dgamma, None


class _AddNormQuant(torch.autograd.Function):
    """model.py:68 / :72 followed by :76-77 -- `x = x + branch; h = rms_norm(x)` -- as one kernel
    (ops.add_rmsnorm_quant_fwd): returns the new residual stream, the norm output and (optionally) its
    quantised pair.  In the backward pass the gradient of the new stream (arriving over the skip path)
    and the norm's input gradient are added inside the norm backward kernel, and that sum is the
    gradient of both `x` and `branch`: neither the forward add nor the fan-in add is a launch."""

    @staticmethod
    def forward(ctx, x, branch, gamma, eps, want_q):
        s, q, sc, h = ops.add_rmsnorm_quant_fwd(x, branch, gamma, eps, want_q=want_q, want_y=True)
        ctx.save_for_backward(s, gamma)
        ctx.eps = eps
        ctx.set_materialize_grads(False)
        if want_q:
            ctx.mark_non_differentiable(q, sc)
            return s, h, q, sc
        return s, h

    @staticmethod
    def backward(ctx, g_s, g_h, *_):
        s, gamma = ctx.saved_tensors
        dgamma = None
        if g_h is None:
            d = g_s
        else:
            d, dgamma = ops.rmsnorm_bwd(s, gamma, g_h.contiguous(), ctx.eps,
                                        addend=None if g_s is None else g_s.contiguous())
        return d, d, dgamma, None, None


class _ExchangePoint(torch.autograd.Function):
    """Identity whose backward tells the gradient buckets to launch the all-reduces that are due
    (dp.GradBuckets.flush): placed on the attention output, so that this happens just before the
    attention backward kernels of a layer -- many short blocks, beside which a collective's kernel gets SMs
    and returns them without holding up a persistent GEMM."""

    @staticmethod
    def forward(ctx, x, buckets):
        ctx.buckets = buckets
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.buckets.flush()
        return g, None


class _QKV(torch.autograd.Function):
    """model.py:63-65 -- q, k, v = h wq, h wk, h wv -- as ONE forward GEMM over the three weights side by side
    (the outputs are column slices of its result: three tensors, no copies), and a backward in which the input gradient dh = gq wq^T + gk wk^T + gv wv^T is ONE GEMM: the three gradients'
    row-wise forms are written side by side into one (tokens, 3 d) matrix by the quantiser itself
    (ops.quantize_rowcol(row_out=...)), the three quantised weights are concatenated the same way, and the
    dgrad contracts over all 3 d columns -- the float32 accumulator does the two adds that autograd would
    otherwise launch on (tokens, d) tensors; the column forms go side by side the same way and ONE wgrad GEMM
    produces the three weight gradients as column slices of its (d, 3 d) result.  Bytes and scales are those of
    the separate calls: a tile never straddles two of the tensors."""

    @staticmethod
    def forward(ctx, h, hq, wq, wk, wv):
        a_q, a_s = hq.rowwise()
        widths = [w.shape[1] for w in (wq, wk, wv)]
        # the three weights side by side, quantised as one matrix (128x128 tiles never straddle two of them):
        # one forward GEMM with 3 d output columns instead of three with d (a (tokens, 1024) x (1024, 1024) launch
        # has 8 contraction blocks per tile and 7 waves: it runs at two thirds of the rate of the wide one)
        # (when the optimiser keeps the three side by side in one flat matrix -- dp.GradBuckets with a grouped
        # entry -- that matrix is read as it is; otherwise they are concatenated)
        sbs = getattr(wq, "side_by_side", None)
        if sbs is not None and len(sbs[1]) == 3 and all(a is b for a, b in zip(sbs[1], (wq, wk, wv))):
            W = sbs[0].detach()
        else:
            W = torch.cat((wq, wk, wv), dim=1)
        W_q, W_s = ops.quantize_block128(W)
        qkv = ops.gemm_fwd(a_q, a_s, W_q, W_s, (128, 128))
        ctx.save_for_backward(h)
        ctx.stash = (hq, W_q, W_s, widths)
        slot = getattr(wq, "grad_slot", None)       # one slot for the three: their gradients side by side (dp.GradSlot)
        ctx.slot = slot if (slot is not None and all(a is b for a, b in zip(slot.params, (wq, wk, wv)))) else None
        outs, off = [], 0
        for n in widths:                                            # column slices: views, no copies
            outs.append(qkv[:, off:off + n].view(*h.shape[:-1], n))
            off += n
        return tuple(outs)

    @staticmethod
    def backward(ctx, *gs):
        (h,) = ctx.saved_tensors
        hq, W_q, W_s, widths = ctx.stash
        M = h.numel() // h.shape[-1]
        N = sum(widths)
        f8 = torch.float8_e4m3fn
        G_q = torch.empty((M, N), dtype=f8, device=h.device)                 # row forms side by side: the dgrad's operand
        G_s = torch.empty((M, N // 128), dtype=torch.float32, device=h.device)
        Gc_q = torch.empty((M, N), dtype=f8, device=h.device)                # column forms side by side: the wgrad's
        Gc_s = torch.empty(((M + 127) // 128, N), dtype=torch.float32, device=h.device)
        off = 0
        for g, n in zip(gs, widths):
            ops.quantize_rowcol(g.reshape(M, n).contiguous(),
                                row_out=(G_q[:, off:off + n], G_s[:, off // 128:(off + n) // 128]),
                                col_out=(Gc_q[:, off:off + n], Gc_s[:, off:off + n]))
            off += n
        dh = ops.gemm_dgrad(G_q, G_s, W_q, W_s, (128, 128))
        x_qc, x_sc = hq.colwise()
        if ctx.slot is not None:                                             # straight into the gradient bucket
            ops.gemm_wgrad(x_qc, x_sc, Gc_q, Gc_s, out=ctx.slot.take())
            ctx.slot.ready()
            return (dh.reshape(h.shape), None, None, None, None)
        dW = ops.gemm_wgrad(x_qc, x_sc, Gc_q, Gc_s)                          # (d, 3 d): the three weight gradients
        dws, off = [], 0
        for n in widths:
            dws.append(dW[:, off:off + n])
            off += n
        return (dh.reshape(h.shape), None, *dws)


class _FusedMLP(torch.autograd.Function):
    """model.py:72 -- `mm(act(mm(h, w_up)), w_down)` -- with both GEMMs and their FP8 backward as in
    fp8.block_scaled_matmul(weight_tile=(128, 128), backward="fp8"), except that the activation is
    never materialised: the down-projection's operand is quantised straight from the up-projection's
    output (ops.act_quantize_rowcol), and in the backward pass the gradient at the pre-activation is
    quantised straight from the down-projection's dgrad output and the saved pre-activation.  Saves
    one bf16 write + read of the (tokens, d_ff) activation each way and two elementwise launches."""

    @staticmethod
    def forward(ctx, h, hq, w_up, w_down, act):
        d = h.shape[-1]
        h2d = h.reshape(-1, d)
        a_q, a_s = hq.rowwise() if hq is not None else ops.quantize_rowwise(h2d)
        wu_q, wu_s = ops.quantize_block128(w_up)
        u = ops.gemm_fwd(a_q, a_s, wu_q, wu_s, (128, 128))                       # pre-activation, bf16
        r_q, r_s, c_q, c_s = ops.act_quantize_rowcol(u, act)                     # act(u): row form now, column form for wgrad
        wd_q, wd_s = ops.quantize_block128(w_down)
        y = ops.gemm_fwd(r_q, r_s, wd_q, wd_s, (128, 128))
        ctx.save_for_backward(h, u)
        ctx.stash = (hq, act, c_q, c_s, wu_q, wu_s, wd_q, wd_s)
        ctx.slots = (getattr(w_up, "grad_slot", None), getattr(w_down, "grad_slot", None))   # dp.GradSlot or None
        return y.reshape(*h.shape[:-1], w_down.shape[1])

    @staticmethod
    def backward(ctx, g):
        h, u = ctx.saved_tensors
        hq, act, c_q, c_s, wu_q, wu_s, wd_q, wd_s = ctx.stash
        g2d = g.reshape(-1, g.shape[-1]).contiguous()
        g_q, g_s, g_qc, g_sc = ops.quantize_rowcol(g2d)
        da = ops.gemm_dgrad(g_q, g_s, wd_q, wd_s, (128, 128))                    # gradient at act(u)
        s_up, s_down = ctx.slots
        dw_down = ops.gemm_wgrad(c_q, c_s, g_qc, g_sc, out=None if s_down is None else s_down.take())
        if s_down is not None:                                                   # written into the gradient bucket
            s_down.ready()
            dw_down = None
        du_q, du_s, du_qc, du_sc = ops.act_quantize_rowcol(u, act + "_bwd", da)  # da * act'(u), quantised, never stored
        dh = ops.gemm_dgrad(du_q, du_s, wu_q, wu_s, (128, 128))
        x_qc, x_sc = hq.colwise() if hq is not None else ops.quantize_colwise(h.reshape(-1, h.shape[-1]))
        dw_up = ops.gemm_wgrad(x_qc, x_sc, du_qc, du_sc, out=None if s_up is None else s_up.take())
        if s_up is not None:
            s_up.ready()
            dw_up = None
        return dh.reshape(h.shape), None, dw_up, dw_down, None


class GPT:
    """Parameters (bf16, model.py:19-54) and forward pass."""

    def __init__(self, cfg: StepConfig, device, seed: int = 0):
        self.cfg = cfg
        g = torch.Generator(device=device).manual_seed(seed)
        std, proj_std = cfg.init_std, cfg.init_std / math.sqrt(2.0 * cfg.n_layers)   # model.py:21-22
        d, h, ff = cfg.d_model, cfg.n_heads * cfg.head_dim, cfg.d_ff

        def normal(shape, s=std):
            return torch.nn.Parameter((torch.randn(shape, device=device, generator=g) * s).to(torch.bfloat16))

        def ones(n):
            return torch.nn.Parameter(torch.ones(n, device=device, dtype=torch.bfloat16))

        self.embed = normal((cfg.vocab_size, d))
        self.pos = normal((cfg.seq_len, d))
        self.layers = []
        for _ in range(cfg.n_layers):
            self.layers.append({
                "norm1": ones(d), "wq": normal((d, h)), "wk": normal((d, h)), "wv": normal((d, h)),
                "wo": normal((h, d), proj_std), "norm2": ones(d), "w_up": normal((d, ff)),
                "w_down": normal((ff, d), proj_std)})
        self.final_norm = ones(d)
        self.unembed = normal((d, cfg.vocab_size))
        self.exchange = None            # gradient buckets with a deferred exchange (data-parallel training): see _ExchangePoint

    def buckets(self, qkv_side_by_side: bool = False):
        """Gradient buckets in the order backward finishes them: head group, layers L-1..0, embeddings.
        qkv_side_by_side: wq, wk, wv of a layer form one entry (a tuple), which dp.GradBuckets lays out as
        column slices of one matrix -- the layout in which ONE weight-gradient GEMM produces all three."""
        out = [[self.unembed, self.final_norm]]
        for lp in reversed(self.layers):
            if qkv_side_by_side:
                out.append([lp["norm1"], (lp["wq"], lp["wk"], lp["wv"]), lp["wo"], lp["norm2"], lp["w_up"], lp["w_down"]])
            else:
                out.append(list(lp.values()))
        out.append([self.embed, self.pos])
        return out

    def parameters(self):
        return [p for b in self.buckets() for p in b]

    def matrices(self):
        """The parameters whose only use is an FP8 linear (model.py:63-72): wq, wk, wv, wo, w_up, w_down."""
        return [lp[n] for lp in self.layers for n in ("wq", "wk", "wv", "wo", "w_up", "w_down")]

    # ---- the mm / norm seam (bench_fp8_norm.py:81-86) -------------------------------------
    def _mm(self, a, w, aq=None):
        m = self.cfg.mm
        if m == "bf16":
            return a @ w
        if m == "fp8":
            return fp8.block_scaled_matmul(a, w, weight_tile=(128, 128), backward="fp8", a_quantized=aq)
        if m == "fp8_ref":
            return fp8.block_scaled_matmul(a, w, a_quantized=aq)
        raise ValueError(f"unknown mm {m!r}")

    def _norm(self, x, w):
        """Returns (y, quantised pair or None)."""
        c = self.cfg
        if c.norm == "fused" and c.mm != "bf16":
            y, q, s = _NormQuant.apply(x, w, c.rms_eps)
            return y, fp8.QuantizedActivation(y, q, s)          # one object for every GEMM this activation feeds
        if c.norm == "pure":
            return kernels._rms_norm_pure(x, w, c.rms_eps), None
        if c.norm == "torch_reference":
            var = x.float().pow(2).mean(-1, keepdim=True)                           # kernels.py:31
            return x * torch.rsqrt(var + c.rms_eps).to(x.dtype) * w, None           # kernels.py:32-33
        return kernels.rms_norm(x, w, c.rms_eps), None

    def _act(self, u):
        return F.gelu(u) if self.cfg.activation == "gelu" else F.relu(u) ** 2      # model.py:72

    def raw_logits(self, ids):
        """model.py:75-96: everything up to the unembedding GEMM (no cap)."""
        c = self.cfg
        B, T = ids.shape
        x = self.embed[ids] + self.pos[:T]                                          # model.py:83
        # With `residual == "fused"` a branch's output is not added where model.py adds it: it waits in
        # `branch` and the norm that follows does the add (same values: one bf16 rounding of x + branch).
        fuse = c.residual == "fused" and c.norm == "fused" and c.mm != "bf16" and c.d_model <= ops.ADD_NORM_MAX_COLS
        branch = None

        def norm_after(x, branch, gamma, want_q=True):
            """(new x, h, quantised h) for `x = x + branch; h = norm(x)`; branch None: no add pending."""
            if branch is None:
                h, hq = self._norm(x, gamma)
                return x, h, hq
            if not fuse:
                x = x + branch
                h, hq = self._norm(x, gamma)
                return x, h, hq
            out = _AddNormQuant.apply(x, branch, gamma, c.rms_eps, want_q)
            return out[0], out[1], (fp8.QuantizedActivation(out[1], out[2], out[3]) if want_q else None)

        for lp in self.layers:
            x, h, hq = norm_after(x, branch, lp["norm1"])                           # model.py:72 (layer before), :76
            if c.qkv == "fused" and c.mm == "fp8" and hq is not None:
                q, k, v = _QKV.apply(h, hq, lp["wq"], lp["wk"], lp["wv"])           # model.py:63-65
            else:
                q, k, v = (self._mm(h, lp[n], hq) for n in ("wq", "wk", "wv"))
            q, k, v = (t.view(B, T, c.n_heads, c.head_dim) for t in (q, k, v))
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
            if self.exchange is not None and torch.is_grad_enabled():
                o = _ExchangePoint.apply(o, self.exchange)
            o = o.transpose(1, 2).reshape(B, T, -1)
            # the attention output feeds one linear: both its quantised forms from one read when a backward pass follows
            oq = fp8.QuantizedActivation.both(o) if (c.mm == "fp8" and torch.is_grad_enabled() and o.shape[-1] % 128 == 0) else None
            branch = self._mm(o, lp["wo"], oq)
            x, h, hq = norm_after(x, branch, lp["norm2"])                           # model.py:68, :77
            if c.mm == "fp8" and c.mlp == "fused":
                branch = _FusedMLP.apply(h, hq, lp["w_up"], lp["w_down"], c.activation)
            else:
                branch = self._mm(self._act(self._mm(h, lp["w_up"], hq)), lp["w_down"])
        x, h, _ = norm_after(x, branch, self.final_norm, want_q=False)              # model.py:72, :93
        return h @ self.unembed                                                     # stays bf16 (bench_fp8_norm.py:86)

    def forward(self, ids):
        logits = self.raw_logits(ids)
        return self.cfg.logit_cap * torch.tanh(logits / self.cfg.logit_cap)         # model.py:97

    def loss(self, ids, targets):
        if self.cfg.loss == "fused":
            return losses.capped_cross_entropy(self.raw_logits(ids), targets, self.cfg.logit_cap)
        logits = self.forward(ids).float()                                          # losses.py:9
        return F.cross_entropy(logits.view(-1, logits.shape[-1]), targets.view(-1))  # losses.py:10-12


class Trainer:
    """train.py:126-137 with the gradient exchange inserted: loss + backward (bucketed
    all-reduce overlapping it), global norm, clip, AdamW.

    graph=True captures the whole step (forward, backward, the bucket all-reduces, clip and
    AdamW) into ONE CUDA graph at the first call and replays it afterwards: the step issues
    about 1900 kernel launches through Python, which leaves the GPU idle a quarter of the time
    when they are launched one by one.  Batches are copied into fixed device buffers before each
    replay; the returned loss and gradient norm are the graph's own output tensors (read them
    before the next step).  Capture needs two eager warm-up steps; parameters and optimizer
    state are restored after them, so a captured run follows the same trajectory as an eager one.
    """

    def __init__(self, cfg: StepConfig, device, world_size: int = 1, seed: int = 0, graph: bool = False,
                 reserve_sms: int | None = None):
        self.cfg, self.device, self.world = cfg, device, world_size
        # With more than one rank the bucket all-reduces run beside the backward pass's GEMMs, which are
        # persistent kernels holding every SM: leave NCCL a few SMs to start on (see tg_set_gemm_reserved_sms).
        if torch.device(device).type == "cuda":
            ops.set_gemm_reserved_sms(RESERVED_SMS_DP if (reserve_sms is None and world_size > 1) else int(reserve_sms or 0))
        self.model = GPT(cfg, device, seed)                     # same seed on every rank: replicated weights
        on_gpu = torch.device(device).type == "cuda"
        self._fused_opt = cfg.optimizer == "fused"
        # Weight gradients written straight into the buckets by their GEMMs (no zero fill of that part, no add
        # into it): needs every use of those weights to be an FP8 linear of this package.  With q, k, v as one
        # weight-gradient GEMM its (d, 3 d) result is the bucket entry itself, so the three are laid out side
        # by side -- parameters and moments too, which is why that needs the flat optimiser state.
        direct = bool(cfg.direct_grads) and on_gpu and cfg.mm == "fp8"
        fused_qkv = cfg.qkv == "fused" and cfg.norm == "fused"
        side_by_side = direct and fused_qkv and self._fused_opt and cfg.flat_parameters
        defer = bool(cfg.defer_exchange) and world_size > 1
        self.buckets = GradBuckets(self.model.buckets(qkv_side_by_side=side_by_side), world_size, defer=defer)
        if defer:
            self.model.exchange = self.buckets
        if direct:
            skip = () if (side_by_side or not fused_qkv) else ("wq", "wk", "wv")    # three slices of one GEMM result: autograd adds them
            self.buckets.enable_direct([lp[n] for lp in self.model.layers for n in ("wq", "wk", "wv", "wo", "w_up", "w_down")
                                        if n not in skip])
        self._want_graph = bool(graph) and on_gpu
        self._graph = None
        if self._fused_opt:
            flat = None
            if cfg.flat_parameters:
                b = self.buckets
                flat = [(fp, fg, ps, (lambda t, bi=bi: b.views(bi, t)))
                        for bi, (fp, fg, ps) in enumerate(zip(b.flatten_parameters(), b.flat, b.params))]
            self.opt = optim.ClippedAdamW(self.model.parameters(), lr=cfg.lr, weight_decay=cfg.weight_decay,
                                          clip_norm=cfg.clip_norm, flat=flat)
        else:
            self.opt = torch.optim.AdamW(self.model.parameters(), lr=cfg.lr, weight_decay=cfg.weight_decay,
                                         betas=(0.9, 0.999), eps=1e-8, fused=on_gpu, capturable=self._want_graph)

    def _eager_step(self, ids, targets):
        self.buckets.zero()
        loss = self.model.loss(ids, targets)
        loss.backward()
        self.buckets.finish()
        if torch.device(self.device).type == "cuda":
            loss = ops.poison_if_failed(loss.detach())        # a GEMM whose bounded wait ran out -> NaN loss
        if self._fused_opt:
            gnorm = self.opt.global_norm(self.buckets.flat)                          # train.py:132
            self.opt.step(gnorm)                                                     # train.py:133-134
            return loss.detach(), gnorm
        gnorm = self.buckets.global_norm()                                           # train.py:132
        scale = torch.clamp(self.cfg.clip_norm / (gnorm + 1e-6), max=1.0)            # optax.clip_by_global_norm
        for f in self.buckets.flat:
            if f.numel():
                f.mul_(scale.to(f.dtype))
        self.opt.step()
        return loss.detach(), gnorm

    def _opt_state_tensors(self):
        if self._fused_opt:
            return self.opt.state_tensors()
        return [t for st in self.opt.state.values() for t in st.values() if torch.is_tensor(t)]

    def _capture(self, ids, targets):
        self._ids, self._tgt = ids.clone(), targets.clone()
        params = self.model.parameters()
        saved_p = [p.detach().clone() for p in params]
        saved_s = {id(t): t.clone() for t in self._opt_state_tensors()}
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):                      # lazy initialisations (optimizer state, kernel attributes, NCCL)
                self._eager_step(self._ids, self._tgt)
        torch.cuda.current_stream().wait_stream(side)
        with torch.no_grad():
            for p, q in zip(params, saved_p):
                p.copy_(q)
            for t in self._opt_state_tensors():
                if id(t) in saved_s:
                    t.copy_(saved_s[id(t)])
                else:
                    t.zero_()                       # state created by the warm-up: back to its initial value
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._loss, self._gnorm = self._eager_step(self._ids, self._tgt)
        self._graph = g

    def step(self, ids, targets):
        if not self._want_graph:
            return self._eager_step(ids, targets)
        if self._graph is None:
            self._capture(ids, targets)
        self._ids.copy_(ids)
        self._tgt.copy_(targets)
        self._graph.replay()
        return self._loss, self._gnorm


_ZIPF_CACHE = {}


def _zipf_table(vocab: int):
    """Token probabilities proportional to 1 / (rank + 10), ranks assigned by a fixed random permutation."""
    if vocab not in _ZIPF_CACHE:
        g = torch.Generator().manual_seed(4321)
        p = 1.0 / (torch.arange(vocab, dtype=torch.float64) + 10.0)
        _ZIPF_CACHE[vocab] = (p / p.sum())[torch.randperm(vocab, generator=g)]
    return _ZIPF_CACHE[vocab]


def synthetic_batch(cfg: StepConfig, batch: int, device, seed: int, learnable=False):
    """Seeded tokens uniform over the vocabulary (data.py:10-11's random windows stand-in).
    `learnable` selects a stream a short run can learn, so that its loss curve falls:
      True / "bigram"  sequences from a fixed random bigram map with 10 % noise (a sharp transition once
                       the map is found: good for "does it train", chaotic in WHEN it falls);
      "zipf"           independent tokens with Zipf-like frequencies (a smooth fall from ln(vocab) to the
                       distribution's entropy: the stream loss-curve comparisons use)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    if not learnable:
        ids = torch.randint(0, cfg.vocab_size, (batch, cfg.seq_len + 1), generator=g)
    elif learnable == "zipf":
        ids = torch.multinomial(_zipf_table(cfg.vocab_size), batch * (cfg.seq_len + 1), replacement=True,
                                generator=g).view(batch, cfg.seq_len + 1)
    else:
        table = torch.randint(0, cfg.vocab_size, (cfg.vocab_size,), generator=torch.Generator().manual_seed(1234))
        ids = torch.empty((batch, cfg.seq_len + 1), dtype=torch.long)
        ids[:, 0] = torch.randint(0, cfg.vocab_size, (batch,), generator=g)
        noise = torch.rand((batch, cfg.seq_len), generator=g) < 0.1
        rnd = torch.randint(0, cfg.vocab_size, (batch, cfg.seq_len), generator=g)
        for t in range(cfg.seq_len):
            ids[:, t + 1] = torch.where(noise[:, t], rnd[:, t], table[ids[:, t]])
    ids = ids.to(device)
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


def step_flops(cfg: StepConfig, tokens: int) -> float:
    """The reference's estimator 6 * L * layer_params * tokens (bench.py:96-102)."""
    d, h, ff = cfg.d_model, cfg.n_heads * cfg.head_dim, cfg.d_ff
    layer_params = 3 * d * h + h * d + 2 * d * ff
    return 6.0 * cfg.n_layers * layer_params * tokens


def bench_train_step(world: int, rank: int, device, dist, steps: int = 20, warmup: int = 3, batch_per_gpu: int = 32,
                     cfg: StepConfig = StepConfig(), graph: bool = True, reserve_sms: int | None = None):
    """Tokens/s of the data-parallel step (the benchmark's training configuration): batch sharded by rank,
    weights replicated, gradients all-reduced per layer bucket over NCCL."""
    # a fresh batch every step (nothing to memorise: uniform tokens hold the loss near ln(vocab))
    batches = [synthetic_batch(cfg, batch_per_gpu, device, seed=100003 * rank + i) for i in range(warmup + steps)]
    graph_error = None
    tr = Trainer(cfg, device, world_size=world, graph=graph, reserve_sms=reserve_sms)
    try:
        for i in range(warmup):
            loss, _ = tr.step(*batches[i])
    except RuntimeError as e:
        if not graph:
            raise
        # capture refused (e.g. by a collective): time the eager step instead and say so
        graph_error, graph = str(e).splitlines()[0][:200], False
        del tr
        torch.cuda.synchronize()
        tr = Trainer(cfg, device, world_size=world, graph=False, reserve_sms=reserve_sms)
        for i in range(warmup):
            loss, _ = tr.step(*batches[i])
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        loss, gnorm = tr.step(*batches[warmup + i])
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tokens = world * batch_per_gpu * cfg.seq_len
    sec = ms / steps * 1e-3
    return {
        "metric": "train_tokens_per_s", "value": tokens / sec, "unit": "tokens/s", "ms_per_step": ms / steps,
        "steps": steps, "warmup": warmup, "loss": float(loss), "grad_norm": float(gnorm),
        "mfu_flops_per_s": step_flops(cfg, tokens) / sec,
        "config": {"layers": cfg.n_layers, "d_model": cfg.d_model, "heads": cfg.n_heads, "d_ff": cfg.d_ff,
                   "vocab": cfg.vocab_size, "seq": cfg.seq_len, "batch_per_gpu": batch_per_gpu, "activation": cfg.activation,
                   "mm": cfg.mm, "norm": cfg.norm, "optimizer": "AdamW lr 3e-4", "parallelism": f"dp{world}", "cuda_graph": bool(graph), "cuda_graph_error": graph_error,
                   "grad_bytes_allreduced": tr.buckets.bytes(), "sms_reserved_for_nccl": ops.set_gemm_reserved_sms(0), "data": "tokens uniform over the vocabulary (seeded)"},
    }


def kernel_breakdown(steps: int = 2, batch_per_gpu: int = 32, cfg: StepConfig = StepConfig(), top: int = 40):
    """Device time per kernel of the (eager) training step on cuda:0, from torch's profiler.
    Prints one line per kernel: ms per step, launches per step, name."""
    from torch.autograd import DeviceType
    from torch.profiler import ProfilerActivity, profile
    dev = torch.device("cuda", 0)
    tr = Trainer(cfg, dev)
    batch = synthetic_batch(cfg, batch_per_gpu, dev, seed=1)
    for _ in range(3):
        tr.step(*batch)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            tr.step(*batch)
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.key_averages() if e.device_type == DeviceType.CUDA),
                key=lambda e: -e.self_device_time_total)
    total = sum(e.self_device_time_total for e in ev) / steps / 1e3
    print(f"device time per step: {total:.2f} ms  ({len(ev)} distinct kernels)")
    for e in ev[:top]:
        ms = e.self_device_time_total / steps / 1e3
        print(f"{ms:8.2f} ms {100 * ms / total:5.1f} % {e.count // steps:5d}  {e.key[:120]}")


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser(description="Training step of the benchmark's training configuration on one GPU")
    ap.add_argument("--kernel-breakdown", action="store_true", help="device time per kernel (torch profiler)")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--no-graph", action="store_true")
    a = ap.parse_args()
    if a.kernel_breakdown:
        kernel_breakdown(steps=min(a.steps, 2))
    else:
        import json
        print(json.dumps(bench_train_step(1, 0, torch.device("cuda", 0), None, steps=a.steps, graph=not a.no_graph)))
