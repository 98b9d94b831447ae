"""Per-kernel microbenchmarks on one GPU (the counterpart of train-gpt's bench_fp8.py GEMM
table and debug_bf16_norm.py `bench_norm`): achieved GB/s for the streaming kernels,
TFLOP/s for the GEMMs, against the algorithmic bytes / FLOPs of each.

    python -m train_gpt_b200.microbench quant  [--rows 32768 --cols 2048]
    python -m train_gpt_b200.microbench norm   [--rows 32768 --cols 2048]
    python -m train_gpt_b200.microbench gemm   [--m 32768 --n 6144 --k 2048 --mode fwd|dgrad|wgrad --tile 128x128|128x1]
    python -m train_gpt_b200.microbench sweep  (square and skinny GEMM shapes)
    python -m train_gpt_b200.microbench sustained [--m .. --n .. --k .. --mode all --seconds 2.5]
                                               (one GEMM back to back for seconds: rate, SM clock, power)

Timing: CUDA events on the launching stream, `--warmup` untimed launches, then `--iters`
samples (ten back-to-back launches each for the streaming kernels, one for a GEMM); operands rotate through enough distinct buffers to exceed the
126 MB L2 between reuses (streaming kernels) or are larger than L2 themselves.  Prints one
JSON object per kernel.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import time

import torch

from . import fp8, ops

L2_BYTES = 126e6


def _time(fn, n_variants, warmup, iters, batch=1):
    """Median and best time of one launch.  `batch` launches go between each pair of events
    (rotating through the input variants) so that host launch gaps do not count against
    kernels that run for tens of microseconds."""
    for i in range(warmup):
        fn(i % n_variants)
    torch.cuda.synchronize()
    ts = []
    k = 0
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(batch):
            fn(k % n_variants)
            k += 1
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) / batch)
    return statistics.median(ts), min(ts)


def _time_graph(fn, warmup, iters, reps=20):
    """Median and best time of one call, with `reps` calls captured in a CUDA graph and the graph
    replayed: for kernels of tens of microseconds, where launching through Python would be what is timed."""
    for _ in range(max(warmup, 2)):
        fn(0)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn(0)
        side.synchronize()
        with torch.cuda.graph(g, stream=side):
            for _ in range(reps):
                fn(0)
    torch.cuda.current_stream().wait_stream(side)
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) / reps)
    return statistics.median(ts), min(ts)


def _outlier_input(rows, cols, n, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    xs = []
    for _ in range(n):
        x = torch.randn(rows, cols, device="cuda", generator=g)
        x = torch.where(torch.rand(rows, cols, device="cuda", generator=g) < 1e-3, x * 50, x)
        xs.append(x.to(torch.bfloat16))
    return xs


EMIT = True      # print one JSON line per kernel (the command-line mode); bench.py collects the dicts instead


def _report(name, ms_med, ms_min, bytes_=None, flops=None, **extra):
    out = {"kernel": name, "ms_median": round(ms_med, 5), "ms_min": round(ms_min, 5)}
    if bytes_ is not None:
        out["algorithmic_MB"] = round(bytes_ / 1e6, 3)
        out["GBps_median"] = round(bytes_ / ms_med / 1e6, 1)
        out["GBps_best"] = round(bytes_ / ms_min / 1e6, 1)
    if flops is not None:
        out["GFLOP"] = round(flops / 1e9, 2)
        out["TFLOPs_median"] = round(flops / ms_med / 1e9, 1)
        out["TFLOPs_best"] = round(flops / ms_min / 1e9, 1)
    out.update(extra)
    if EMIT:
        print(json.dumps(out), flush=True)
    return out


def bench_quant(rows, cols, warmup, iters, acts=True):
    E = rows * cols
    n = max(2, int(L2_BYTES * 2 // (E * 2)) + 1)
    xs = _outlier_input(rows, cols, n)
    out = []
    m, b = _time(lambda i: ops.quantize_rowwise(xs[i]), n, warmup, iters, batch=10)
    out.append(_report("quantize_rowwise", m, b, bytes_=3.03125 * E, shape=[rows, cols]))
    m, b = _time(lambda i: ops.quantize_colwise(xs[i]), n, warmup, iters, batch=10)
    out.append(_report("quantize_colwise", m, b, bytes_=3.03125 * E, shape=[rows, cols]))
    m, b = _time(lambda i: ops.quantize_block128(xs[i]), n, warmup, iters, batch=10)
    out.append(_report("quantize_block128", m, b, bytes_=(3.0 + 4.0 / 16384) * E, shape=[rows, cols]))
    m, b = _time(lambda i: ops.quantize_rowcol(xs[i]), n, warmup, iters, batch=10)
    out.append(_report("quantize_rowcol", m, b, bytes_=(2.0 + 2 * 1.03125) * E, shape=[rows, cols]))
    if not acts:
        return out
    # the MLP activation (or its gradient) computed inside the same pass
    gs = [(torch.randn(rows, cols, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(n)]
    for act in ("relu2", "gelu"):
        m, b = _time(lambda i: ops.act_quantize_rowcol(xs[i], act), n, warmup, iters, batch=10)
        out.append(_report(f"act_quantize_rowcol[{act}]", m, b, bytes_=(2.0 + 2 * 1.03125) * E, shape=[rows, cols]))
        m, b = _time(lambda i: ops.act_quantize_rowcol(xs[i], act + "_bwd", gs[i]), n, warmup, iters, batch=10)
        out.append(_report(f"act_quantize_rowcol[{act}_bwd]", m, b, bytes_=(4.0 + 2 * 1.03125) * E, shape=[rows, cols]))
    return out


def bench_loss(rows, vocab, warmup, iters):
    """Capped-logit cross-entropy: forward reads the logits and writes the tanh values (4 B per
    element), backward rewrites them as the gradient in place (4 B per element)."""
    E = rows * vocab
    g = torch.Generator(device="cuda").manual_seed(0)
    xs = [(torch.randn(rows, vocab, device="cuda", generator=g) * 4).to(torch.bfloat16) for _ in range(2)]
    tg = torch.randint(0, vocab, (rows,), device="cuda", generator=g).to(torch.int32)
    m, b = _time(lambda i: ops.softcap_ce_fwd(xs[i], tg, 15.0), 2, warmup, iters)
    _report("softcap_ce_fwd", m, b, bytes_=4.0 * E + 12 * rows, shape=[rows, vocab])
    _, lse, th = ops.softcap_ce_fwd(xs[0], tg, 15.0)
    ths = [th, th.clone()]
    # timing the in-place form would feed gradients back in as tanh values: time the out-of-place form
    m, b = _time(lambda i: ops.softcap_ce_bwd(ths[i], tg, lse, None, 15.0), 2, warmup, iters)
    _report("softcap_ce_bwd", m, b, bytes_=4.0 * E + 8 * rows, shape=[rows, vocab])


def bench_norm(rows, cols, warmup, iters):
    E = rows * cols
    n = max(2, int(L2_BYTES * 2 // (E * 2)) + 1)
    xs = _outlier_input(rows, cols, n)
    gs = [torch.randn(rows, cols, device="cuda").to(torch.bfloat16) for _ in range(n)]
    gamma = (1 + 0.1 * torch.randn(cols, device="cuda")).to(torch.bfloat16)
    eps = 1e-6
    out = []
    m, b = _time(lambda i: ops.rmsnorm_quant_fwd(xs[i], gamma, eps), n, warmup, iters, batch=10)
    out.append(_report("rmsnorm_quant_fwd", m, b, bytes_=3.03125 * E + 2 * cols, shape=[rows, cols]))
    m, b = _time(lambda i: ops.rmsnorm_fwd(xs[i], gamma, eps), n, warmup, iters, batch=10)
    out.append(_report("rmsnorm_fwd", m, b, bytes_=4.0 * E + 2 * cols, shape=[rows, cols]))
    m, b = _time(lambda i: ops.rmsnorm_bwd(xs[i], gamma, gs[i], eps), n, warmup, iters, batch=10)
    out.append(_report("rmsnorm_bwd", m, b, bytes_=6.0 * E + 4 * cols, shape=[rows, cols]))
    if cols <= ops.ADD_NORM_MAX_COLS:
        # the residual add folded in: x, res read; sum, y, q (+ scales) written / x, g, addend read; dx written
        m, b = _time(lambda i: ops.add_rmsnorm_quant_fwd(xs[i], gs[i], gamma, eps), n, warmup, iters, batch=10)
        out.append(_report("add_rmsnorm_quant_fwd", m, b, bytes_=9.03125 * E + 2 * cols, shape=[rows, cols]))
        m, b = _time(lambda i: ops.rmsnorm_bwd(xs[i], gamma, gs[i], eps, addend=gs[(i + 1) % n]), n, warmup, iters, batch=10)
        out.append(_report("rmsnorm_bwd_add", m, b, bytes_=8.0 * E + 4 * cols, shape=[rows, cols]))
    return out


def _gemm_case(M, N, K, mode, tile, warmup, iters, student_t=False):
    """M tokens, linear layer (K -> N).  mode picks which of the layer's three GEMMs runs."""
    g = torch.Generator(device="cuda").manual_seed(0)
    if student_t:
        # Student-t(3) = N(0,1) / sqrt(chi2(3)/3), drawn on the device
        chi = sum(torch.randn(M, K, device="cuda", generator=g) ** 2 for _ in range(3)) / 3.0
        x = (torch.randn(M, K, device="cuda", generator=g) / chi.sqrt()).to(torch.bfloat16)
        del chi
    else:
        x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(K, N, device="cuda", generator=g)).to(torch.bfloat16)
    gr = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    st = ops.new_status("cuda")
    if mode == "fwd":
        a_q, a_s = ops.quantize_rowwise(x)
        w_q, w_s = fp8.quantize_weight(w, tile)
        fn = lambda i: ops.gemm_fwd(a_q, a_s, w_q, w_s, tile, status=st)
    elif mode == "dgrad":
        g_q, g_s = ops.quantize_rowwise(gr)
        w_q, w_s = ops.quantize_rowwise(w) if tile == (128, 1) else ops.quantize_block128(w)
        fn = lambda i: ops.gemm_dgrad(g_q, g_s, w_q, w_s, tile, status=st)
    elif mode == "wgrad_blockgrad":
        x_q, x_s = ops.quantize_colwise(x)
        g_q, g_s = ops.quantize_block128(gr)
        fn = lambda i: ops.gemm_wgrad(x_q, x_s, g_q, g_s, status=st, grad_tile=(128, 128))
    else:
        x_q, x_s = ops.quantize_colwise(x)
        g_q, g_s = ops.quantize_colwise(gr)
        fn = lambda i: ops.gemm_wgrad(x_q, x_s, g_q, g_s, status=st)
    # a launch of a few tens of microseconds is timed from a CUDA graph (20 launches per replay)
    m, b = _time_graph(fn, warmup, iters) if 2.0 * M * N * K < 1e11 else _time(fn, 1, warmup, iters)
    if int(st.item()) != 0:
        raise RuntimeError(f"GEMM bounded wait expired, status {int(st.item())}")
    return _report(f"gemm_{mode}", m, b, flops=2.0 * M * N * K, tokens=M, K=K, N=N,
                   weight_tile=f"{tile[0]}x{tile[1]}", pct_of_4500=round(2.0 * M * N * K / m / 1e9 / 45.0, 1))


def _gemm_fn(M, N, K, mode, tile):
    """Quantised operands of one layer GEMM and a closure that launches it."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(K, N, device="cuda", generator=g)).to(torch.bfloat16)
    gr = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    st = ops.new_status("cuda")
    if mode == "fwd":
        a_q, a_s = ops.quantize_rowwise(x)
        w_q, w_s = fp8.quantize_weight(w, tile)
        return (lambda: ops.gemm_fwd(a_q, a_s, w_q, w_s, tile, status=st)), st
    if mode == "dgrad":
        g_q, g_s = ops.quantize_rowwise(gr)
        w_q, w_s = ops.quantize_rowwise(w) if tile == (128, 1) else ops.quantize_block128(w)
        return (lambda: ops.gemm_dgrad(g_q, g_s, w_q, w_s, tile, status=st)), st
    x_q, x_s = ops.quantize_colwise(x)
    g_q, g_s = ops.quantize_colwise(gr)
    return (lambda: ops.gemm_wgrad(x_q, x_s, g_q, g_s, status=st)), st


def _sample_while(fn, seconds):
    """Runs fn back to back for `seconds` while nvidia-smi samples the GPU every 50 ms (reading only);
    returns launches, ms per launch and the medians of SM clock and power over the last three quarters."""
    dev = torch.cuda.current_device()
    smi = subprocess.Popen(
        ["nvidia-smi", "-i", str(dev), "--query-gpu=clocks.sm,power.draw,clocks_event_reasons.sw_power_cap,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.sw_thermal_slowdown", "--format=csv,noheader,nounits",
         "-lms", "50"], stdout=subprocess.PIPE, text=True)
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0, n = time.time(), 0
    e0.record()
    while time.time() - t0 < seconds:
        for _ in range(50):
            fn()
        n += 50
        torch.cuda.synchronize()
    e1.record()
    e1.synchronize()
    ms = e0.elapsed_time(e1) / n
    smi.terminate()
    rows = [l.split(", ") for l in smi.stdout.read().strip().splitlines() if l.count(",") >= 4]
    rows = rows[len(rows) // 4:]
    clk = [float(r[0]) for r in rows] or [0.0]
    pw = [float(r[1]) for r in rows] or [0.0]
    return dict(launches=n, ms_per_launch=round(ms, 4), sm_mhz_median=statistics.median(clk), sm_mhz_min=min(clk),
                power_w_median=round(statistics.median(pw), 1), samples=len(rows),
                sw_power_cap=sum(r[2].strip() == "Active" for r in rows),
                slowdown=sum(r[3].strip() == "Active" or r[4].strip() == "Active" for r in rows))


def bench_sustained(M, N, K, modes, tile, seconds):
    """What a GEMM sustains once the board sits at its power limit: the same launch back to back for
    `seconds`, with the SM clock and the power the board settled at, and a cuBLAS bf16 8192^3 loop for
    scale.  `tensor_busy` is the rate over what 148 SMs x 16384 FLOP per cycle give at that clock."""
    out = []
    for mode in modes:
        fn, st = _gemm_fn(M, N, K, mode, tile)
        r = _sample_while(fn, seconds)
        if int(st.item()) != 0:
            raise RuntimeError(f"GEMM bounded wait expired, status {int(st.item())}")
        r.update(kernel=f"gemm_{mode}", tokens=M, K=K, N=N)
        r["TFLOPs"] = round(2.0 * M * N * K / r["ms_per_launch"] / 1e9, 1)
        if r["sm_mhz_median"] > 0:
            r["tensor_busy"] = round(r["TFLOPs"] * 1e12 / (148 * 16384 * r["sm_mhz_median"] * 1e6), 3)
        out.append(r)
        if EMIT:
            print(json.dumps(r), flush=True)
        time.sleep(1.0)
    a = torch.randn(8192, 8192, device="cuda").to(torch.bfloat16)
    r = _sample_while(lambda: torch.mm(a, a), seconds)
    r.update(kernel="cublas_bf16_8192x8192x8192")
    r["TFLOPs"] = round(2.0 * 8192 ** 3 / r["ms_per_launch"] / 1e9, 1)
    if r["sm_mhz_median"] > 0:
        r["tensor_busy"] = round(r["TFLOPs"] * 1e12 / (148 * 8192 * r["sm_mhz_median"] * 1e6), 3)
    out.append(r)
    if EMIT:
        print(json.dumps(r), flush=True)
    return out


def bench_sweep(tile=(128, 128), warmup=5, iters=30):
    """The shape sweep of the benchmark configurations (Student-t(3) activations): squares
    M = N = K in {1024 .. 16384}, then skinny M in {16, 64, 256} with K = N = 8192, each as forward,
    dgrad and wgrad.  A skinny case streams the 67 MB weight once, so it also reports that as GB/s."""
    out = []
    for n in (1024, 2048, 4096, 8192, 16384):
        for mode in ("fwd", "dgrad", "wgrad"):
            out.append(_gemm_case(n, n, n, mode, tile, warmup, max(5, iters // 3), student_t=True))
    for m in (16, 64, 256):
        for mode in ("fwd", "dgrad", "wgrad"):
            r = _gemm_case(m, 8192, 8192, mode, tile, warmup, iters, student_t=True)
            # fwd / dgrad read the e4m3 weight (K*N bytes); wgrad writes the bf16 gradient (2*K*N bytes)
            stream = 8192 * 8192 * (2 if mode == "wgrad" else 1)
            r["weight_stream_GBps"] = round(stream / r["ms_median"] / 1e6, 1)
            out.append(r)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["quant", "norm", "gemm", "loss", "sweep", "sustained"])
    ap.add_argument("--vocab", type=int, default=50304)
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--cols", type=int, default=2048)
    ap.add_argument("--m", type=int, default=32768)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--mode", default="fwd", choices=["fwd", "dgrad", "wgrad", "wgrad_blockgrad", "all"])
    ap.add_argument("--tile", default="128x128", choices=["128x128", "128x1"])
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--seconds", type=float, default=2.5)
    a = ap.parse_args()
    tile = (128, 128) if a.tile == "128x128" else (128, 1)
    if a.what == "quant":
        bench_quant(a.rows, a.cols, a.warmup, a.iters)
    elif a.what == "norm":
        bench_norm(a.rows, a.cols, a.warmup, a.iters)
    elif a.what == "loss":
        bench_loss(a.rows, a.vocab, a.warmup, a.iters)
    elif a.what == "gemm":
        for mode in (["fwd", "dgrad", "wgrad"] if a.mode == "all" else [a.mode]):
            _gemm_case(a.m, a.n, a.k, mode, tile, a.warmup, a.iters)
    elif a.what == "sustained":
        bench_sustained(a.m, a.n, a.k, ["fwd", "dgrad", "wgrad"] if a.mode == "all" else [a.mode], tile, a.seconds)
    else:
        bench_sweep(tile, a.warmup, a.iters)


if __name__ == "__main__":
    main()
