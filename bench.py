"""Benchmark of the quantization hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload: NF4 block-64 quantization of every linear weight of a LLaMA-2-7B-shaped model
(225 bf16 tensors, 6 607 077 376 elements, ~N(0, 0.02) from per-tensor seeds), packed two codes
per byte plus one fp32 scale per block.  A step is one pass over all tensors of this rank.
Algorithmic traffic: 2 B read + 0.5 B codes + 4/64 B scale = 2.5625 B per element (16.93 GB).

  value   GB/s of algorithmic traffic with inputs resident in HBM (CUDA events, max over ranks)
  e2e     same metric through HostPipeline: pinned host tensors in, packed host results out
  With N > 1 the tensors are partitioned over the ranks (strong scaling, no collective).

``--impl reference`` times the CPU restatement of the upstream ops (oracle/voyager_oracle.py) on
the host cores for a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BYTES_PER_ELEM = 2.0 + 0.5 + 4.0 / 64.0
BLOCK = 64
LAYER = [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)]
WORKLOAD = "cfg3: NF4 block-64 quantization of LLaMA-2-7B-shaped linear weights (225 bf16 tensors)"
# DRAM bytes (read + write) one launch of the headline kernel moves over the full single-GPU
# workload, from a profiler capture of a one-layer launch scaled by the elements processed.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 16.32e9


def model_shapes(layers=32):
    """All 225 tensors; ``layers < 32`` gives a reduced model (no lm_head) for profiler captures."""
    if layers >= 32:
        return LAYER * 32 + [(32000, 4096)]
    return LAYER * layers


def make_tensor(idx, shape, device, rows=None):
    """Tensor ``idx`` of the model: randn * 0.02 in bf16 from its own seed (so the values do not
    depend on how many GPUs share the model); ``rows`` keeps a row range."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(2_000_000 + idx)
    w = (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    if rows is not None and rows != (0, shape[0]):
        w = w[rows[0]:rows[1]].contiguous()
    return w


# Written between timed iterations of the additional measurements: larger than L2 (126 MB), and long enough on the
# device (about 0.16 ms) for the host to have queued the next call before it ends, so that the events bracket device
# time and not the Python path of the op.
FLUSH_BYTES = int(os.environ.get("VOYAGER_B200_BENCH_FLUSH_MB", "1024")) << 20


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while a timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-i", str(self.gpu), "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.p is None:
            return out
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, smax, reasons = [], [], set()
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); smax.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(smax), reasons=sorted(reasons), samples=len(sm))
        return out


def oracle_module():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import voyager_oracle
    return voyager_oracle


def cpu_time_oracle(tensors_cpu, repeats=1):
    """Seconds for the CPU restatement (calculate_mx_qparam + quantize with the NF4 index table,
    as convert_pt2e calls them) over ``tensors_cpu`` with all host threads; best of ``repeats``."""
    import torch
    vo = oracle_module()
    tab = vo.value_table("nf4")
    idx, _, _ = vo.index_table(tab)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        for w in tensors_cpu:
            s = vo.mx_scale(w, (-1,), BLOCK, 1.0, False)
            vo.quantize(w, s, None, (-1,), BLOCK, idx)
        best = min(best, time.perf_counter() - t0)
    return best, torch.get_num_threads()


def parity_sample(tensors, results, qmap, max_tensors=4, max_rows=1024):
    """Compares up to ``max_tensors`` packed results (first ``max_rows`` rows each; rows are
    independent) with the CPU oracle.  Returns (elements checked, mismatching codes + scales)."""
    import numpy as np
    import torch
    vo = oracle_module()
    tab = torch.from_numpy(qmap.view(np.int16).copy()).view(torch.bfloat16)
    idx_tab, _, _ = vo.index_table(tab)
    n = len(tensors)
    pick = sorted({0, n // 3, (2 * n) // 3, n - 1})[:max_tensors]
    checked = bad = 0
    for i in pick:
        rows = min(max_rows, tensors[i].shape[0])
        w = tensors[i][:rows].cpu()
        s_ref = vo.mx_scale(w, (-1,), BLOCK, 1.0, False).float()
        c_ref = vo.quantize(w, s_ref.to(w.dtype), None, (-1,), BLOCK, idx_tab).to(torch.uint8)
        codes = results[i].codes[:rows].cpu()
        got = torch.stack([codes & 0xF, codes >> 4], dim=-1).reshape(w.shape)
        bad += int((got != c_ref).sum()) + int((results[i].scale[:rows].cpu().view(torch.int32) != s_ref.view(torch.int32)).sum())
        checked += w.numel()
    return checked, bad


def _timed_flushed(torch, fn, iters, flush):
    """Median and best milliseconds of ``fn`` (CUDA events on the current stream), three warm-up
    calls, the L2 overwritten before every timed call."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts), min(ts)


def _timing_context(torch, flush, copy_bytes=None, iters=50, read_bytes=None):
    """What the timing method itself contributes to a small launch, measured with the vendor's kernels under the same
    bracket (L2 overwritten, event, call, event): ``floor_us`` is a 4-byte fill (a launch that moves nothing), and
    ``copy_us`` a device-to-device ``copy_`` that reads and writes ``copy_bytes`` in total.  Means over ``iters``
    calls (the event clock ticks in steps of about a microsecond, so medians of short launches are quantised).
    ``read_us``: torch's ``amax`` over ``read_bytes`` of fp32, a read-only pass of the size of the cfg1 tensor."""
    one = torch.zeros(1, device=flush.device)

    def mean_us(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.fmean(ts) * 1e3

    ctx = {"floor_us": mean_us(one.zero_), "floor_is": "torch fill of 4 bytes, same bracket"}
    if copy_bytes:
        a = torch.empty(int(copy_bytes) // 2, dtype=torch.uint8, device=flush.device)
        b = torch.empty_like(a)
        ctx["copy_us"] = mean_us(lambda: b.copy_(a))
        ctx["copy_is"] = f"torch copy_ moving {int(copy_bytes)} bytes in total (half read, half written), same bracket"
        del a, b
    if read_bytes:
        r = torch.empty(int(read_bytes) // 4, dtype=torch.float32, device=flush.device).normal_()
        ctx["read_us"] = mean_us(lambda: torch.amax(r))
        ctx["read_is"] = f"torch amax over {int(read_bytes)} bytes of fp32 (a read-only pass by the vendor's reduction), same bracket"
        del r
    return ctx


def _bits_differ(torch, got, want):
    """Number of elements whose values differ (NaN == NaN, -0 != +0)."""
    a, b = got.detach().cpu().contiguous(), want.detach().cpu().contiguous()
    if a.shape != b.shape or a.dtype != b.dtype:
        return max(a.numel(), b.numel())
    it = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[a.element_size()]
    ai, bi = a.view(it), b.view(it)
    if a.is_floating_point():
        both_nan = torch.isnan(a) & torch.isnan(b)
        return int(((ai != bi) & ~both_nan).sum())
    return int((ai != bi).sum())


def _timed_graph(torch, fns, iters, flush):
    """Median time per call of ``fns`` captured together in one CUDA graph (L2 flushed before every replay);
    None when the calls cannot be captured."""
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for f in fns:
                f()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            keep = [f() for f in fns]                            # noqa: F841  (outputs live as long as the graph)
        for _ in range(2):
            graph.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); graph.replay(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / len(fns))
        return statistics.median(ts)
    except Exception as e:  # noqa: BLE001
        sys.stderr.write(f"graph timing skipped: {type(e).__name__}: {e}\n")
        torch.cuda.synchronize()
        return None


def run_extras(dev, iters=20):
    """The other configurations of the baseline on one GPU, each timed (CUDA events, L2 flushed
    between iterations) and compared with the CPU oracle on the same tensors: cfg1 (MXINT8 block 32
    of fp32 [4096, 4096] with outliers), cfg2 (posit8 per output channel over the 54 ResNet-50-shaped
    weights, one fused launch), cfg4 (per-row 16-level quantile codebooks of a Student-t weight),
    cfg5 (MX linear 8192 x 11008 x 4096), and the reference's composite of torch operators run on
    this GPU for the headline sample.  GB/s are algorithmic bytes / time; ``frac`` is of the measured peak."""
    import numpy as np
    import torch
    import voyager_compiler_b200 as vb
    from voyager_compiler_b200 import codebook, gemm_native, model_quant as mq

    vo = oracle_module()
    Q = torch.ops.quantized_ops
    peaks, kind = measured_peaks()
    flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
    out = {"peak_kind": kind, "l2": f"{FLUSH_BYTES >> 20} MB written between timed iterations"}
    out["timing_context"] = _timing_context(torch, flush, copy_bytes=25_502_912 * 9, iters=iters, read_bytes=4096 * 4096 * 4)

    def tab(name):
        return torch.from_numpy(vb.tables.build_table(name).view(np.int16).copy()).view(torch.bfloat16)

    def hbm(name, fn, nbytes, mismatches=None, rotating=None, **more):
        med, best = _timed_flushed(torch, fn, iters, flush)
        gbs = nbytes / med / 1e6
        out[name] = {"ms": med, "value": gbs, "unit": "GB/s", "best": nbytes / best / 1e6, "algorithmic_bytes": int(nbytes),
                     "frac": gbs / peaks["hbm_gbs"], **({"mismatches": mismatches} if mismatches is not None else {}), **more}
        if rotating:
            # the same call on `len(rotating)` different input buffers (together larger than L2, so every launch reads
            # cold data), replayed as ONE CUDA graph: launch gaps and event overhead are shared by all of them
            g_ms = _timed_graph(torch, rotating, iters, flush)
            if g_ms is not None:
                out[name]["graph_of"] = len(rotating)
                out[name]["graph_ms_per_call"] = g_ms
                out[name]["graph_frac"] = nbytes / g_ms / 1e6 / peaks["hbm_gbs"]

    # ---- cfg1
    torch.manual_seed(0)
    x1 = torch.randn(4096, 4096)
    x1[torch.rand_like(x1) < 0.001] *= 50
    q8 = tab("int8")
    s_ref, c_ref = vo.quantize_mx(x1, q8, (-1,), 32, 127.0, True)
    d_ref = vo.dequantize(c_ref, s_ref, None, (-1,), 32)
    xg, q8g = x1.to(dev), q8.to(dev)
    n = x1.numel()
    s, c = Q.quantize_mx(xg, q8g, (-1,), 32, 127.0, True)
    d = Q.dequantize(c, s, None, (-1,), 32)
    R = 8                                                        # rotating copies: 8 x 67 MB of input
    xr = [xg] + [xg.clone() for _ in range(R - 1)]
    cr = [c] + [c.clone() for _ in range(R - 1)]
    hbm("cfg1_quantize_mx_fp32", lambda: Q.quantize_mx(xg, q8g, (-1,), 32, 127.0, True), n * (4 + 4 + 4 / 32),
        _bits_differ(torch, s, s_ref) + _bits_differ(torch, c, c_ref),
        rotating=[(lambda t=t: Q.quantize_mx(t, q8g, (-1,), 32, 127.0, True)) for t in xr])
    hbm("cfg1_dequantize_fp32", lambda: Q.dequantize(c, s, None, (-1,), 32), n * (4 + 4 + 4 / 32), _bits_differ(torch, d, d_ref),
        rotating=[(lambda t=t: Q.dequantize(t, s, None, (-1,), 32)) for t in cr])
    sq = Q.calculate_mx_qparam(xg, (-1,), 32, 127.0, True)
    hbm("cfg1_calculate_mx_qparam_fp32", lambda: Q.calculate_mx_qparam(xg, (-1,), 32, 127.0, True), n * (4 + 4 / 32),
        _bits_differ(torch, sq, s_ref), rotating=[(lambda t=t: Q.calculate_mx_qparam(t, (-1,), 32, 127.0, True)) for t in xr])
    plans = [mq.MXQuantPlan([t], q8, 32, 127.0, True, code_bits=8, want_exp=True) for t in xr]
    plan1 = plans[0]
    packed = [pl.run()[0] for pl in plans]
    p1 = packed[0]
    torch.cuda.synchronize()
    bad = _bits_differ(torch, p1.scale, s_ref) + int((p1.codes.cpu().view(torch.int8).float() != c_ref).sum()) + \
        int((p1.exp_e8.cpu() != torch.log2(s_ref).clamp(-127, 127).to(torch.int8)).sum())
    hbm("cfg1_packed_int8_codes_e8_exponents", plan1.run, n * (4 + 1 + 4 / 32 + 1 / 32), bad, rotating=[pl.run for pl in plans])
    dp = mq.dequantize_packed(p1, torch.float32, use_exponent=True)
    hbm("cfg1_dequantize_packed_int8_e8_to_fp32", lambda: mq.dequantize_packed(p1, torch.float32, use_exponent=True),
        n * (1 + 1 / 32 + 4), int((dp.cpu() != d_ref).sum()),
        rotating=[(lambda pk=pk: mq.dequantize_packed(pk, torch.float32, use_exponent=True)) for pk in packed])
    for pl in plans:
        pl.close()
    del xg, s, c, d, sq, p1, dp, plan1, plans, packed, xr, cr

    # ---- cfg2
    torch.manual_seed(1)
    rn = []
    for shp in resnet50_weight_shapes():
        t = torch.empty(shp)
        torch.nn.init.kaiming_normal_(t, mode="fan_in")
        rn.append(t)
    qp = tab("posit8_1")
    rg = [t.to(dev) for t in rn]
    n2 = sum(t.numel() for t in rn)
    plan2 = mq.ChannelQuantPlan(rg, qp, 4096.0, want_codes=True, want_dequant=True, want_values=True)
    res2 = plan2.run()
    torch.cuda.synchronize()
    bad = 0
    for w, r in zip(rn, res2):
        sc = vo.channel_scale(w, 4096.0)
        qv = vo.quantize(w, sc, None, None, None, qp)
        bad += _bits_differ(torch, r.scale, sc) + _bits_differ(torch, r.values, qv) + _bits_differ(torch, r.dequant, vo.dequantize(qv, sc))
        ok = ~torch.isnan(qv)
        bad += int((r.levels[r.codes.cpu().long().clamp(max=r.levels.numel() - 1)][ok] != qv.float()[ok]).sum())
    del plan2, res2
    plan2 = mq.ChannelQuantPlan(rg, qp, 4096.0, want_codes=True, want_dequant=True)
    more_plans = [mq.ChannelQuantPlan([t.clone() for t in rg], qp, 4096.0, want_codes=True, want_dequant=True) for _ in range(3)]
    hbm("cfg2_posit8_per_channel_54_tensors_codes_and_dequant", plan2.run, n2 * 9, bad, launches_per_pass=1,
        rotating=[plan2.run] + [pl.run for pl in more_plans])
    for pl in more_plans:
        pl.close()
    del more_plans
    plan2b = mq.ChannelQuantPlan(rg, qp, 4096.0, want_values=True, want_dequant=False)
    hbm("cfg2_posit8_per_channel_54_tensors_values", plan2b.run, n2 * 8)
    del plan2, plan2b, rg, rn

    # ---- cfg4
    torch.manual_seed(3)
    w4 = torch.distributions.StudentT(5.0).sample((11008, 4096)) * 0.02
    w4g = w4.to(dev)
    lv = codebook.row_quantile_levels(w4g, 16)
    rows = 256
    qq = (2 * torch.arange(16, dtype=torch.float32) + 1) / 32
    lv_ref = torch.quantile(w4[:rows], qq, dim=-1).t().contiguous()
    bad_fit = int((lv[:rows].cpu() != lv_ref).sum())
    n4 = w4.numel()
    hbm("cfg4_row_quantile_fit16", lambda: codebook.row_quantile_levels(w4g, 16), n4 * 4 + lv.numel() * 4, bad_fit,
        rows_checked=rows)
    for rule, nm in ((True, "reference_rule"), (False, "fp32_rule")):
        idx, val = codebook.row_codebook_quantize(w4g, lv, reference_rule=rule)
        i_ref, v_ref = vo.row_codebook(w4[:rows], lv[:rows].cpu(), reference_rule=rule)
        bad = int((idx[:rows].cpu() != i_ref).sum()) + _bits_differ(torch, val[:rows], v_ref)
        hbm(f"cfg4_row_codebook16_search_{nm}", lambda: codebook.row_codebook_quantize(w4g, lv, reference_rule=rule),
            n4 * 9 + lv.numel() * 4, bad, rows_checked=rows)
    del w4g, w4, idx, val, lv

    # ---- cfg5
    torch.manual_seed(4)
    M, N, K = 8192, 11008, 4096
    x5 = torch.randn(M, K).bfloat16()
    w5 = (torch.randn(N, K) * 0.02).bfloat16()
    xg, wg = x5.to(dev), w5.to(dev)
    ws, wq = Q.quantize_mx(wg, q8g, (-1,), 32, 127.0, True)
    xs, xq = Q.quantize_mx(xg, q8g, (-1,), 32, 127.0, True)
    xs_ref, xq_ref = vo.quantize_mx(x5[:512], q8, (-1,), 32, 127.0, True)
    bad_q = _bits_differ(torch, xs[:512], xs_ref) + _bits_differ(torch, xq[:512], xq_ref)
    y_ref = vo.linear_mx(xq.cpu(), wq.cpu(), None, input_scale=xs.cpu(), weight_scale=ws.cpu(), block_size=32).double()
    flops = 2.0 * M * N * K

    def tc(name, fn, **more):
        y = fn()
        torch.cuda.synchronize()
        rel = float(((y.cpu().double() - y_ref).norm() / y_ref.norm()).item())
        med, best = _timed_flushed(torch, fn, iters, flush)
        out[name] = {"ms": med, "value": flops / med / 1e9, "unit": "TFLOP/s", "best": flops / best / 1e9, "flops": flops,
                     "frac": flops / med / 1e9 / peaks["bf16_tflops"], "frac_of_sustained": flops / med / 1e9 / peaks["bf16_tflops_sustained"],
                     "rel_frobenius_error_vs_oracle": rel, "tolerance": 1e-2, "within_tolerance": rel <= 1e-2, **more}

    tc("cfg5_linear_mx", lambda: Q.linear_mx(xq, wq, None, input_scale=xs, weight_scale=ws, block_size=32))
    os.environ["VOYAGER_B200_GEMM"] = "fused"
    tc("cfg5_linear_mx_fused_staging", lambda: Q.linear_mx(xq, wq, None, input_scale=xs, weight_scale=ws, block_size=32))
    os.environ.pop("VOYAGER_B200_GEMM", None)
    tc("cfg5_quantize_mx_plus_linear_mx", lambda: Q.linear_mx(Q.quantize_mx(xg, q8g, (-1,), 32, 127.0, True)[1], wq, None,
                                                              input_scale=xs, weight_scale=ws, block_size=32),
       activation_quantize_mismatches=bad_q, rows_checked=512)
    tc("cfg5_linear_mx_dynamic_one_pass_activation",
       lambda: gemm_native.linear_mx_dynamic(xg, wq, None, qmap=q8g, weight_scale=ws, block_size=32, quant_max=127.0))
    # ---- fp32 operands of the same linear on a quarter of the rows: tf32 contraction (fp32 result)
    Mf = 2048
    xs_f, xq_f = Q.quantize_mx(xg[:Mf].float(), q8g, (-1,), 32, 127.0, True)
    ws_f, wq_f = ws.float(), wq.float()
    yf_ref = y_ref[:Mf]
    yf = Q.linear_mx(xq_f, wq_f, None, input_scale=xs_f, weight_scale=ws_f, block_size=32)
    torch.cuda.synchronize()
    rel_f = float(((yf.cpu().double() - yf_ref).norm() / yf_ref.norm()).item())
    med, best = _timed_flushed(torch, lambda: Q.linear_mx(xq_f, wq_f, None, input_scale=xs_f, weight_scale=ws_f, block_size=32), iters, flush)
    out["linear_mx_fp32_operands_tf32_2048_rows"] = {
        "ms": med, "value": flops / 4 / med / 1e9, "unit": "TFLOP/s", "flops": flops / 4, "rel_frobenius_error_vs_oracle": rel_f,
        "tolerance": 1e-2, "within_tolerance": rel_f <= 1e-2, "note": "reference: the bf16 oracle result of the same codes and scales"}
    out["cfg5_status_ok"] = gemm_native.gemm_status(dev) == 0
    del xg, wg, xq, wq, xs, ws, xq_f, wq_f, xs_f, ws_f

    # ---- conv2d_mx: one ResNet-50 layer, MXINT8 block 32 along the channels,
    # NHWC; implicit GEMM (default), patch matrix + GEMM, decode + vendor convolution; checked against the oracle
    torch.manual_seed(6)
    xc = torch.randn(32, 28, 28, 128).bfloat16()
    wc = (torch.randn(3, 3, 128, 128) * 0.05).bfloat16()
    xcs, xcq = vo.quantize_mx(xc, q8, (3,), 32, 127.0, True)
    wcs, wcq = vo.quantize_mx(wc, q8, (2,), 32, 127.0, True)
    yc_ref = vo.conv2d_mx(xcq.float(), wcq.float(), None, 1, 1, 1, 1, input_scale=xcs.float(), weight_scale=wcs.float(),
                          block_size=32, layout="nhwc").double()
    cargs = [t.to(dev) for t in (xcq, wcq, xcs, wcs)]
    cflops = 2.0 * 32 * 28 * 28 * 128 * 128 * 9

    def conv():
        return Q.conv2d_mx(cargs[0], cargs[1], None, (1, 1), (1, 1), (1, 1), 1, input_scale=cargs[2], weight_scale=cargs[3],
                           block_size=32, layout="nhwc")
    for form in ("native", "patches", "vendor"):
        os.environ["VOYAGER_B200_CONV"] = form
        yc = conv()
        torch.cuda.synchronize()
        rel = float(((yc.cpu().double() - yc_ref).norm() / yc_ref.norm()).item())
        med, best = _timed_flushed(torch, conv, iters, flush)
        name = {"native": "implicit_gemm", "patches": "patch_matrix_plus_gemm", "vendor": "decode_plus_vendor_convolution"}[form]
        out[f"conv2d_mx_3x3_128to128_28x28_batch32_{name}"] = {
            "ms": med, "value": cflops / med / 1e9, "unit": "TFLOP/s", "flops": cflops, "rel_frobenius_error_vs_oracle": rel,
            "tolerance": 1e-2, "within_tolerance": rel <= 1e-2}
    os.environ.pop("VOYAGER_B200_CONV", None)
    out["conv_status_ok"] = gemm_native.gemm_status(dev) == 0

    # ---- the reference's composite of torch operators on this GPU (one layer of the headline workload)
    nf4 = vo.value_table("nf4")
    idx_tab = vo.index_table(nf4)[0].to(dev)
    sample = [make_tensor(i, shp, dev) for i, shp in enumerate(LAYER)]
    ns = sum(t.numel() for t in sample)

    def composite():
        for w in sample:
            sc = vo.mx_scale(w, (-1,), BLOCK, 1.0, False)
            vo.quantize(w, sc, None, (-1,), BLOCK, idx_tab)
    med, best = _timed_flushed(torch, composite, 5, flush)
    out["composite_on_gpu"] = {"ms": med, "value": ns * BYTES_PER_ELEM / med / 1e6, "unit": "GB/s",
                               "sample": f"one layer: {len(sample)} of 225 tensors, {ns} elements",
                               "what": "calculate_mx_qparam + quantize as chains of torch operators on CUDA tensors (the device-agnostic upstream formulation)"}
    return out


EXTRAS_MULTI_LIMIT_S = 180


def run_extras_multi(dev, world, rank, iters=10):
    """cfg5 sharded by output columns over the ranks (every rank calls this): the local GEMM alone,
    GEMM + NCCL all-gather, and the GEMM whose epilogue stores its columns into every rank's copy of
    Y over NVLink.  Times are CUDA events, max over ranks; results are compared with the one-GPU op."""
    import numpy as np
    import torch
    import torch.distributed as dist
    import voyager_compiler_b200 as vb
    from voyager_compiler_b200 import parallel as par

    Q = torch.ops.quantized_ops
    peaks, _ = measured_peaks()
    flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
    M, N, K = 8192, 11008, 4096
    g = torch.Generator(device=dev); g.manual_seed(4)
    x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    q8 = torch.from_numpy(vb.tables.build_table("int8").view(np.int16).copy()).view(torch.bfloat16).to(dev)
    ws, wq = Q.quantize_mx(w, q8, (-1,), 32, 127.0, True)
    xs, xq = Q.quantize_mx(x, q8, (-1,), 32, 127.0, True)
    wq_r, ws_r = par.shard_weight(wq, ws, rank, world)
    y1 = Q.linear_mx(xq, wq, None, input_scale=xs, weight_scale=ws, block_size=32)
    flops = 2.0 * M * N * K
    out = {"shards": par.column_shards(N, world)}

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            dist.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t.item()))
        return statistics.median(ts)

    def entry(ms, same=None):
        e = {"ms": ms, "value": flops / ms / 1e9, "unit": "TFLOP/s (whole job)", "frac_of_n_gpu_peak": flops / ms / 1e9 / (peaks["bf16_tflops"] * world)}
        if same is not None:
            e["equals_single_gpu_result"] = same
        return e

    out["cfg5_single_gpu_linear_mx"] = entry(timed(lambda: Q.linear_mx(xq, wq, None, input_scale=xs, weight_scale=ws, block_size=32)))
    out["cfg5_column_shard_gemm_only"] = entry(timed(lambda: Q.linear_mx(xq, wq_r, None, input_scale=xs, weight_scale=ws_r, block_size=32)))
    lin = par.ColumnParallelLinearMX(wq_r, ws_r, N, 32)          # all-gather in pieces, overlapped with the next piece's GEMM
    y = lin(xq, xs)
    out["cfg5_column_parallel_nccl_all_gather"] = entry(timed(lambda: lin(xq, xs)), bool(torch.equal(y, y1)))
    out["cfg5_column_parallel_nccl_all_gather"]["pieces"] = len(lin.pieces)
    ok = torch.ones(1, device=dev)
    p2p = None
    try:
        p2p = par.P2PColumnParallelLinearMX(wq_r, ws_r, N, 32, M)
    except Exception as e:  # noqa: BLE001  (peer-mapped memory may be unavailable on a given box)
        ok.zero_()
        out["cfg5_column_parallel_peer_store_epilogue"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)         # every rank takes the same branch
    if bool(ok.item()):
        y2 = p2p(xq, xs)
        torch.cuda.synchronize()
        same = bool(torch.equal(y2, y1))
        e = entry(timed(lambda: p2p(xq, xs)), same)
        e["status_ok"] = p2p.status() == 0
        out["cfg5_column_parallel_peer_store_epilogue"] = e
    elif "cfg5_column_parallel_peer_store_epilogue" not in out:
        out["cfg5_column_parallel_peer_store_epilogue"] = {"unavailable": "another rank could not map peer memory"}
    return out


def run_reference(args):
    """CPU arm: rank 0 alone times the oracle port on a bounded sample per step."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 to its workers: the CPU arm is to use every host thread it can
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if torch.get_num_threads() < cores:
        torch.set_num_threads(cores)
    torch.manual_seed(2)
    sample_shapes = LAYER                         # one transformer layer: 7 tensors
    ws = [(torch.randn(s) * 0.02).to(torch.bfloat16) for s in sample_shapes]
    elems = sum(w.numel() for w in ws)
    for _ in range(max(args.warmup, 1) if args.warmup < 2 else 2):
        cpu_time_oracle(ws)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_time_oracle(ws)
    dt = (time.perf_counter() - t0) / args.steps
    gbs = elems * BYTES_PER_ELEM / dt / 1e9
    sample = f"one layer per step: {len(ws)} of 225 tensors, {elems} elements"
    line = {
        "impl": "reference", "metric": "nf4_whole_model_quantize_hbm_gbps", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    import voyager_compiler_b200 as vb
    from voyager_compiler_b200 import model_quant as mq

    shapes = model_shapes(args.layers)
    sizes = [r * c for r, c in shapes]
    shard = mq.shard_plan(sizes, [r for r, _ in shapes], world)[rank]
    tensors = [make_tensor(i, shapes[i], dev, (b, e)) for i, b, e in shard]
    my_elems = sum(t.numel() for t in tensors)
    total_elems = sum(sizes)
    qmap = vb.tables.build_table("nf4")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the pass is prepared once (outputs, descriptors, launch shape); a step is then one library
    # call = one kernel launch over every tensor of this rank
    plan = mq.MXQuantPlan(tensors, qmap, BLOCK, 1.0, False, code_bits=4)
    step = plan.run

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = vb._lib.launch_count()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    enqueue_s = 0.0
    evs[0].record()
    for k in range(args.steps):
        h0 = time.perf_counter()
        step()
        enqueue_s += time.perf_counter() - h0
        evs[k + 1].record()
    barrier()
    launches = vb._lib.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    total_ms = evs[0].elapsed_time(evs[-1])
    per_step = [evs[k].elapsed_time(evs[k + 1]) for k in range(args.steps)]
    # per rank: mean device time of a step (one launch) and mean host time spent queueing it
    mine = torch.tensor([total_ms, statistics.mean(per_step), enqueue_s / args.steps * 1e3, float(my_elems)],
                        device=dev, dtype=torch.float64)
    if world > 1:
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
    else:
        every = [mine]
    every = [e.tolist() for e in every]
    total_ms = max(e[0] for e in every)
    ms_per_step = total_ms / args.steps
    value = total_elems * BYTES_PER_ELEM / (ms_per_step * 1e-3) / 1e9

    # parity of what was just timed: a few of this rank's outputs against the CPU oracle
    checked, mismatches = parity_sample(tensors, plan.results, qmap)
    par = torch.tensor([checked, mismatches], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(par, op=dist.ReduceOp.SUM)
    checked, mismatches = int(par[0].item()), int(par[1].item())
    plan.close()
    del plan

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"kernel_only": True, "layers": args.layers, "ms_per_step": ms_per_step, "value": value,
                              "unit": "GB/s", "gpu_launches": int(launches), "parity_checked": checked,
                              "mismatches": mismatches, "kernel_ms": [e[1] for e in every]}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end: pinned host tensors in, packed pinned host results out
    e2e_steps = max(1, min(args.steps, 3))
    host = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in tensors]
    for h, t in zip(host, tensors):
        h.copy_(t)
    host_out = [(torch.empty(tuple(t.shape[:-1]) + (t.shape[-1] // 2,), dtype=torch.uint8, pin_memory=True),
                 torch.empty(tuple(t.shape[:-1]) + (t.shape[-1] // BLOCK,), dtype=torch.float32, pin_memory=True))
                for t in tensors]
    del tensors
    torch.cuda.empty_cache()
    pipe = mq.HostPipeline(dev, qmap, BLOCK, 1.0, False, code_bits=4)
    pipe.run(host, host_out)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        pipe.run(host, host_out)
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    hb = torch.tensor([float(pipe.h2d_bytes), float(pipe.d2h_bytes)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(hb, op=dist.ReduceOp.SUM)
    e2e_ms = float(t.item()) / e2e_steps
    e2e_value = total_elems * BYTES_PER_ELEM / (e2e_ms * 1e-3) / 1e9

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        # one launch per step and rank: the roofline entry describes the SLOWEST rank's launch
        slow = max(range(world), key=lambda r: every[r][1])
        kernel_ms, slow_elems = every[slow][1], every[slow][3]
        achieved = slow_elems * BYTES_PER_ELEM / (kernel_ms * 1e-3) / 1e9
        line = {
            "metric": "nf4_whole_model_quantize_hbm_gbps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "elements": total_elems, "block": BLOCK, "codes": "4-bit packed",
                       "scales": "fp32 per block", "sharding": f"layer-wise over {world} rank(s), lm_head split by rows",
                       "l2": "inputs (13.2 GB) far exceed L2; no flush needed", "whole_model_quant_seconds": ms_per_step * 1e-3},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "h2d_bytes_per_step": int(hb[0].item()), "d2h_bytes_per_step": int(hb[1].item())},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "mx_fast2_kernel<bf16, amax, LUT, pack4>", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH * slow_elems / total_elems,
                         "algorithmic_bytes_per_launch": slow_elems * BYTES_PER_ELEM, "launch_ms": kernel_ms, "rank": slow},
            "kernel_ms": [e[1] for e in every], "enqueue_ms": [e[2] for e in every],
            "parity_checked": checked, "mismatches": mismatches,
        }
        if world == 1:
            # the pinned host copies of the e2e leg are the very tensors the GPU quantized
            secs, cores = cpu_time_oracle(host, repeats=1)
            n = sum(w.numel() for w in host)
            line["cpu_baseline"] = {"value": n * BYTES_PER_ELEM / secs / 1e9, "unit": "GB/s", "cores": cores,
                                    "kind": "port", "seconds": secs,
                                    "sample": f"all {len(host)} tensors of the workload once ({n} elements)"}
    extra = None
    if not args.no_extras:
        if world > 1:
            # The headline line must come out whatever the additional multi-GPU measurements do: if they raise on
            # one rank the others wait in a collective for ever, so every rank arms a timer that prints the line
            # (rank 0) and leaves the process; a rank that raises prints and leaves at once.
            import threading

            def bail(reason):
                if rank == 0:
                    line["extra"] = {"error": reason}
                    print(json.dumps(line), flush=True)
                sys.stdout.flush()
                os._exit(0)
            timer = threading.Timer(EXTRAS_MULTI_LIMIT_S, bail, args=(f"multi-GPU extras did not finish within {EXTRAS_MULTI_LIMIT_S} s",))
            timer.daemon = True
            timer.start()
            try:
                extra = run_extras_multi(dev, world, rank)
            except Exception as e:  # noqa: BLE001
                import traceback
                traceback.print_exc()
                timer.cancel()
                bail(f"{type(e).__name__}: {e}"[:300])
            timer.cancel()
        elif rank == 0:
            del host, host_out
            torch.cuda.empty_cache()
            try:
                extra = run_extras(dev)
            except Exception as e:  # noqa: BLE001  (the headline line is still to be printed)
                import traceback
                traceback.print_exc()
                extra = {"error": f"{type(e).__name__}: {e}"[:300]}
    if rank == 0:
        if extra is not None:
            line["extra"] = extra
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def conv_cases(res, timed, Q, qmap, g, dev, steps, only=None):
    """conv2d_mx: ResNet-50-shaped bf16 convolutions, batch 32, MXINT8 codes with block 32 along the channels
    (plain bf16 for the 3-channel stem).  Per case: the library's default form (implicit GEMM where the
    channel count allows, else patch matrix + GEMM), the patch-matrix form forced, the default with the decoded
    weight matrix rebuilt on every call, and the vendor convolution on the same operands decoded by this
    library's kernels.  Two grouped cases (ResNeXt-style 32 groups) close the list."""
    import torch
    from voyager_compiler_b200 import conv_native
    conv_shapes = [("stem_7x7s2_3to64_224", 3, 224, 64, 7, 2, 3, 1), ("l1_3x3_64to64_56", 64, 56, 64, 3, 1, 1, 1),
                   ("l1_1x1_64to256_56", 64, 56, 256, 1, 1, 0, 1), ("l2_3x3_128to128_28", 128, 28, 128, 3, 1, 1, 1),
                   ("l3_3x3_256to256_14", 256, 14, 256, 3, 1, 1, 1), ("l4_1x1_1024to2048_s2_14", 1024, 14, 2048, 1, 2, 0, 1),
                   ("l4_3x3_512to512_7", 512, 7, 512, 3, 1, 1, 1),
                   ("resnext_3x3_256to256_g32_56", 256, 56, 256, 3, 1, 1, 32), ("resnext_3x3_1024to1024_g32_14", 1024, 14, 1024, 3, 1, 1, 32)]
    for name, C, HW, O, k, s_, p_, groups in conv_shapes:
        for layout in ("nhwc", "nchw"):
            if only and only not in f"{name}_{layout}":
                continue
            xc = torch.randn(32, C, HW, HW, generator=g, device=dev).bfloat16()
            wc = (torch.randn(O, C // groups, k, k, generator=g, device=dev) * 0.05).bfloat16()
            w_hwio = layout == "nhwc" and groups == 1
            if layout == "nhwc":
                xc = xc.permute(0, 2, 3, 1).contiguous()
            if w_hwio:
                wc = wc.permute(2, 3, 1, 0).contiguous()
            kw = {}
            bs = min(32, C // groups)
            if C % 32 == 0 and bs >= 8:
                ax_x, ax_w = ((3,) if layout == "nhwc" else (1,)), ((2,) if w_hwio else (1,))
                xs_c, xc = Q.quantize_mx(xc, qmap, ax_x, bs, 127.0, True)
                ws_c, wc = Q.quantize_mx(wc, qmap, ax_w, bs, 127.0, True)
                kw = dict(input_scale=xs_c, weight_scale=ws_c, block_size=bs)
            Ho = (HW + 2 * p_ - k) // s_ + 1
            cflops = 2.0 * 32 * Ho * Ho * O * (C // groups) * k * k
            call = lambda: Q.conv2d_mx(xc, wc, None, (s_, s_), (p_, p_), (1, 1), groups, layout=layout, **kw)
            os.environ["VOYAGER_B200_CONV"] = "native"
            med_n, _ = timed(call, steps)

            def call_cold():                     # the weight matrix rebuilt on every call, as the vendor arm decodes it
                conv_native._weight_cache.clear()
                return call()
            med_c, _ = timed(call_cold, steps)
            entry = {"ms": med_n, "tflops": cflops / med_n / 1e9, "ms_weight_not_cached": med_c,
                     "form": "implicit" if conv_native.implicit_ok(C, groups) else "patches"}
            if groups == 1:
                os.environ["VOYAGER_B200_CONV"] = "patches"
                entry["patches_ms"], _ = timed(call, steps)
            os.environ["VOYAGER_B200_CONV"] = "vendor"
            med_v, _ = timed(call, steps)
            os.environ["VOYAGER_B200_CONV"] = "native"
            entry.update(vendor_ms=med_v, vendor_tflops=cflops / med_v / 1e9)
            res[f"conv2d_mx_{name}_{layout}"] = entry


def run_linear_f32(args):
    """linear_mx on fp32 operands (MXINT8 codes and power-of-two scales in fp32 containers): the tf32 contraction,
    ``--m`` rows (default 8192; the bench's extra block uses 2048) x 11008 x 4096.  One JSON line."""
    import torch
    import voyager_compiler_b200 as vb
    from voyager_compiler_b200.gemm_native import gemm_status

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    M, N, K = args.m, 11008, 4096
    g = torch.Generator(device=dev); g.manual_seed(4)
    Q = torch.ops.quantized_ops
    qmap = torch.from_numpy(vb.tables.build_table("int8").view("int16").copy()).view(torch.bfloat16).to(dev)
    xs, xq = Q.quantize_mx(torch.randn(M, K, generator=g, device=dev), qmap, (-1,), 32, 127.0, True)
    ws, wq = Q.quantize_mx(torch.randn(N, K, generator=g, device=dev) * 0.02, qmap, (-1,), 32, 127.0, True)
    flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
    fn = lambda: Q.linear_mx(xq, wq, None, input_scale=xs, weight_scale=ws, block_size=32)
    y = fn()
    ref = torch.nn.functional.linear((xq * xs.repeat_interleave(32, 1)).double(), (wq * ws.repeat_interleave(32, 1)).double())
    rel = float(((y.double() - ref).norm() / ref.norm()).item())
    med, best = _timed_flushed(torch, fn, args.steps, flush)
    peaks, kind = measured_peaks()
    flops = 2.0 * M * N * K
    print(json.dumps({"workload": f"linear_mx, fp32 operands, {M} x {N} x {K}: decode kernels + tf32 tcgen05 GEMM", "ms": med,
                      "tflops": flops / med / 1e9, "best_tflops": flops / best / 1e9,
                      "frac_of_half_the_measured_bf16_peak": flops / med / 1e9 / (peaks["bf16_tflops"] / 2), "peak_kind": kind,
                      "rel_frobenius_error_vs_fp64_product": rel, "gemm_status": gemm_status(dev)}))


def run_conv(args):
    """The conv2d_mx cases alone (see conv_cases): one JSON line."""
    import torch
    import voyager_compiler_b200 as vb

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev); g.manual_seed(4)
    Q = torch.ops.quantized_ops
    qmap = torch.from_numpy(vb.tables.build_table("int8").view("int16").copy()).view(torch.bfloat16).to(dev)
    flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts), min(ts)

    res = {}
    sampler = ClockSampler(dev.index or 0); sampler.start()
    conv_cases(res, timed, Q, qmap, g, dev, args.steps, args.only)
    clocks = sampler.stop()
    from voyager_compiler_b200.gemm_native import gemm_status
    print(json.dumps({"workload": "conv2d_mx, ResNet-50 / ResNeXt-shaped layers, batch 32, bf16 MXINT8 block 32", "results": res,
                      "gemm_status": gemm_status(dev), "clocks": clocks}))


def run_linear(args):
    """cfg5: MX-quantized linear, X[8192,4096] x W[11008,4096]^T, MXINT8 block 32 (single GPU).
    Times the quantize_mx of the activations, the fused GEMM, the plain GEMM (dequantize kernels +
    TMA-fed GEMM) and the vendor bf16 GEMM on pre-dequantised operands for comparison."""
    import torch
    import voyager_compiler_b200 as vb
    from voyager_compiler_b200 import gemm_native

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    M, N, K = args.m, 11008, 4096
    g = torch.Generator(device=dev); g.manual_seed(4)
    x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    Q = torch.ops.quantized_ops
    qmap = torch.from_numpy(vb.tables.build_table("int8").view("int16").copy()).view(torch.bfloat16).to(dev)
    ws, wq = Q.quantize_mx(w, qmap, (-1,), 32, 127.0, True)
    xs, xq = Q.quantize_mx(x, qmap, (-1,), 32, 127.0, True)
    flops = 2.0 * M * N * K
    flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts), min(ts)

    res = {}
    sampler = ClockSampler(dev.index or 0); sampler.start()
    for mode in ("fused", "plain"):
        os.environ["VOYAGER_B200_GEMM"] = mode
        med, best = timed(lambda: Q.linear_mx(xq, wq, None, input_scale=xs, weight_scale=ws, block_size=32), args.steps)
        res[mode] = {"ms": med, "tflops": flops / med / 1e9, "best_tflops": flops / best / 1e9}
    os.environ.pop("VOYAGER_B200_GEMM", None)
    xd, wd = Q.dequantize(xq, xs, None, (-1,), 32), Q.dequantize(wq, ws, None, (-1,), 32)
    med, best = timed(lambda: torch.nn.functional.linear(xd, wd), args.steps)
    res["vendor_bf16_gemm_only"] = {"ms": med, "tflops": flops / med / 1e9, "best_tflops": flops / best / 1e9}
    med, best = timed(lambda: Q.quantize_mx(x, qmap, (-1,), 32, 127.0, True), args.steps)
    res["quantize_mx_activations"] = {"ms": med, "gbs": (x.numel() * (2 + 2 + 2 / 32)) / med / 1e6}
    med, best = timed(lambda: Q.linear_mx(Q.quantize_mx(x, qmap, (-1,), 32, 127.0, True)[1], wq, None, input_scale=xs,
                                          weight_scale=ws, block_size=32), args.steps)
    res["quantize_plus_linear"] = {"ms": med, "tflops": flops / med / 1e9}
    # the same value with the activation's codes * scale written straight into the GEMM operand (one pass over x)
    med, best = timed(lambda: gemm_native.linear_mx_dynamic(x, wq, None, qmap=qmap, weight_scale=ws, block_size=32, quant_max=127.0),
                      args.steps)
    res["quantize_plus_linear_one_pass_activation"] = {"ms": med, "tflops": flops / med / 1e9, "best_tflops": flops / best / 1e9}
    # packed operands: int8 bytes + bf16 scales, conversion inside the GEMM's operand staging
    from voyager_compiler_b200 import model_quant as mq
    (px,) = mq.quantize_tensors_mx([x], qmap, 32, 127.0, True, code_bits=8)
    (pw,) = mq.quantize_tensors_mx([w], qmap, 32, 127.0, True, code_bits=8)
    med, best = timed(lambda: gemm_native.linear_mx_packed(px, pw), args.steps)
    res["packed_int8_fused"] = {"ms": med, "tflops": flops / med / 1e9, "best_tflops": flops / best / 1e9}
    med, best = timed(lambda: gemm_native.linear_mx_packed(
        mq.quantize_tensors_mx([x], qmap, 32, 127.0, True, code_bits=8)[0], pw), args.steps)
    res["quantize_packed_plus_packed_linear"] = {"ms": med, "tflops": flops / med / 1e9}
    # outlier side path: 0.1 % of the activations x 50, split off above a threshold, sparse correction added
    xo = x.clone()
    xo[torch.rand(M, K, generator=g, device=dev) < 0.001] *= 50
    thr = 8.0
    med, best = timed(lambda: Q.quantize_mx_outlier(xo, qmap, (-1,), 32, 127.0, True, None, None, thr, 0.01, 0), args.steps)
    res["quantize_mx_outlier"] = {"ms": med, "gbs": (xo.numel() * (2 + 2 + 2 + 2 / 32)) / med / 1e6}
    od, oi, op_, os_, oc = Q.quantize_mx_outlier(xo, qmap, (-1,), 32, 127.0, True, None, None, thr, 0.01, 0)
    nnz = int(op_[-1].item())
    med, best = timed(lambda: Q.spmm_csr(od, oi, op_, wq, ws, None, 32, "kc"), args.steps)
    res["spmm_csr"] = {"ms": med, "nnz": nnz}
    med, best = timed(lambda: Q.linear_mx(oc, wq, None, input_scale=os_, weight_scale=ws, block_size=32, A_data=od,
                                          A_indices=oi, A_indptr=op_), args.steps)
    res["linear_mx_with_outliers"] = {"ms": med, "tflops": flops / med / 1e9, "nnz": nnz}
    conv_cases(res, timed, Q, qmap, g, dev, args.steps)
    # GPTQ compensation of one [4096, 4096] weight on the NF4 / block-64 grid (Hessian of 8192 synthetic tokens):
    # the column walk alone (64 block launches + 63 trailing updates) and the whole entry point
    import types
    from voyager_compiler_b200 import gptq as gq, qtables
    wg = torch.randn(4096, 4096, generator=g, device=dev) * 0.02
    xg = torch.randn(8192, 4096, generator=g, device=dev) * (0.2 + 2 * torch.rand(4096, generator=g, device=dev))
    hg = xg.t() @ xg
    nf4 = qtables.table_handle("nf4", dev).lut16.view(torch.bfloat16)
    fake = types.SimpleNamespace(qmap=nf4, scale_qmap=None, quant_max=1.0, block_size=64, ch_axis=-1)
    hinv_g = gq.hessian_inverse_chol(hg.clone(), 8192, 0.01)
    sal_g = hg.diagonal().clone()
    med, best = timed(lambda: gq.walk(wg, hinv_g, sal_g, nf4, None, 1.0, 64, False), max(3, args.steps // 4))
    res["gptq_walk_4096x4096_nf4_b64"] = {"ms": med, "best_ms": best, "columns_per_s": 4096 / med * 1e3}
    med, best = timed(lambda: gq.compensate_weight(wg, hg, 8192, fake, 0.01), max(3, args.steps // 4))
    res["gptq_compensate_weight_4096x4096_nf4_b64"] = {"ms": med, "best_ms": best}
    clocks = sampler.stop()
    peaks, kind = measured_peaks()
    ok = gemm_native.gemm_status(dev) == 0
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        # column-sharded linear: every rank owns a slice of W's rows, X is replicated, Y is all-gathered
        import torch.distributed as dist
        from voyager_compiler_b200 import parallel as par
        dist.init_process_group("nccl", device_id=dev)
        rank = dist.get_rank()
        wq_r, ws_r = par.shard_weight(wq, ws, rank, world)

        def timed_dist(fn, iters):
            for _ in range(3):
                fn()
            ts = []
            for _ in range(iters):
                flush.zero_()
                dist.barrier(); torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ts.append(float(t.item()))
            return statistics.median(ts)

        ms_local = timed_dist(lambda: Q.linear_mx(xq, wq_r, None, input_scale=xs, weight_scale=ws_r, block_size=32), args.steps)
        ms_full = timed_dist(lambda: par.column_parallel_linear_mx(xq, xs, wq_r, ws_r, N, 32), args.steps)
        y = par.column_parallel_linear_mx(xq, xs, wq_r, ws_r, N, 32)
        y1 = Q.linear_mx(xq, wq, None, input_scale=xs, weight_scale=ws, block_size=32)
        same = bool(torch.equal(y, y1))
        res[f"column_parallel_{world}gpu"] = {"gemm_only_ms": ms_local, "gemm_only_tflops": flops / ms_local / 1e9,
                                              "gemm_plus_allgather_ms": ms_full, "tflops": flops / ms_full / 1e9,
                                              "shards": par.column_shards(N, world), "equals_single_gpu_result": same}
        try:
            p2p = par.P2PColumnParallelLinearMX(wq_r, ws_r, N, 32, M)
            ms_p2p = timed_dist(lambda: p2p(xq, xs), args.steps)
            y2 = p2p(xq, xs)
            torch.cuda.synchronize()
            res[f"p2p_fused_gather_{world}gpu"] = {"ms": ms_p2p, "tflops": flops / ms_p2p / 1e9,
                                                   "equals_single_gpu_result": bool(torch.equal(y2, y1)),
                                                   "status_ok": p2p.status() == 0}
        except Exception as e:  # noqa: BLE001  (symmetric memory may be unavailable on a given box)
            res[f"p2p_fused_gather_{world}gpu"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        dist.destroy_process_group()
        if rank != 0:
            return
    print(json.dumps({"workload": f"cfg5: MX linear M={M} N={N} K={K} MXINT8 block 32", "results": res, "clocks": clocks,
                      "status_ok": ok, "peak_bf16_tflops": peaks.get("bf16_tflops"),
                      "peak_bf16_tflops_sustained": peaks.get("bf16_tflops_sustained"), "peak_kind": kind,
                      "frac_fused_of_burst_peak": res["fused"]["tflops"] / peaks.get("bf16_tflops", 1590.0)}))


def resnet50_weight_shapes():
    """The 53 convolution weights and the classifier weight of the standard ResNet-50 (25 502 912 elements)."""
    shapes = [(64, 3, 7, 7)]
    inplanes = 64
    for planes, blocks in ((64, 3), (128, 4), (256, 6), (512, 3)):
        for b in range(blocks):
            shapes += [(planes, inplanes, 1, 1), (planes, planes, 3, 3), (planes * 4, planes, 1, 1)]
            if b == 0:
                shapes.append((planes * 4, inplanes, 1, 1))
            inplanes = planes * 4
    shapes.append((1000, 2048))
    return shapes


def run_channel(args):
    """cfg2 alone: the 54 ResNet-50-shaped weight tensors, posit8_1 per output channel (scale = channel
    maximum / 4096), code byte + dequantized fp32 from one prepared launch; ``--steps`` timed launches with
    ``FLUSH_BYTES`` written in between.  Small enough for a full profiler capture of the kernel."""
    import torch
    import voyager_compiler_b200 as vb
    from voyager_compiler_b200 import model_quant as mq

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
    qp = torch.from_numpy(vb.tables.build_table("posit8_1").view("int16").copy()).view(torch.bfloat16).to(dev)
    torch.manual_seed(1)
    ws = []
    for shp in resnet50_weight_shapes():
        t = torch.empty(shp, device=dev)
        torch.nn.init.kaiming_normal_(t, mode="fan_in")
        ws.append(t)
    n = sum(t.numel() for t in ws)
    plan = mq.ChannelQuantPlan(ws, qp, 4096.0, want_codes=True, want_dequant=True)
    for _ in range(max(args.warmup, 1)):
        plan.run()
    torch.cuda.synchronize()
    ts = []
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); plan.run(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    peaks, kind = measured_peaks()
    med = statistics.median(ts)
    ctx = _timing_context(torch, flush, copy_bytes=n * 9, iters=min(args.steps, 50))
    print(json.dumps({"workload": "cfg2: posit8_1 per output channel, 54 ResNet-50-shaped tensors, codes + dequantized fp32",
                      "elements": n, "bytes_per_launch": n * 9, "us_per_launch": med * 1e3, "mean_us_per_launch": statistics.fmean(ts) * 1e3,
                      "gbs": n * 9 / med / 1e6,
                      "frac_of_measured_hbm_peak": n * 9 / med / 1e6 / peaks["hbm_gbs"], "peak_kind": kind,
                      "timing_context": ctx, "same_bytes_copy_frac_of_measured_hbm_peak": n * 9 / ctx["copy_us"] / 1e3 / peaks["hbm_gbs"],
                      "steps": args.steps, "channel_status": vb._lib.lib.vq_channel_status()}))
    plan.close()


def run_elementwise(args):
    """cfg1 / cfg2 / cfg4-shaped element-wise measurements on one GPU (GB/s of algorithmic traffic,
    L2 flushed between iterations)."""
    import torch
    import voyager_compiler_b200 as vb
    from voyager_compiler_b200 import model_quant as mq

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    Q = torch.ops.quantized_ops
    flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)

    def tab(name):
        return torch.from_numpy(vb.tables.build_table(name).view("int16").copy()).view(torch.bfloat16).to(dev)

    def timed(fn, nbytes, iters=args.steps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        med = statistics.median(ts)
        return {"ms": med, "gbs": nbytes / med / 1e6, "best_gbs": nbytes / min(ts) / 1e6}

    peaks, kind = measured_peaks()
    res = {}
    # cfg1: fp32 [4096,4096], outliers, MXINT8 block 32, power-of-two scales
    g = torch.Generator(device=dev); g.manual_seed(0)
    x = torch.randn(4096, 4096, generator=g, device=dev)
    x[torch.rand(4096, 4096, generator=g, device=dev) < 0.001] *= 50
    n = x.numel()
    q8 = tab("int8")
    s, c = Q.quantize_mx(x, q8, (-1,), 32, 127.0, True)
    res["cfg1_quantize_mx_fp32_dropin"] = timed(lambda: Q.quantize_mx(x, q8, (-1,), 32, 127.0, True), n * (4 + 4 + 4 / 32))
    res["cfg1_dequantize_fp32"] = timed(lambda: Q.dequantize(c, s, None, (-1,), 32), n * (4 + 4 + 4 / 32))
    res["cfg1_quantize_mx_packed_int8_e8"] = timed(
        lambda: mq.quantize_tensors_mx([x], q8, 32, 127.0, True, code_bits=8, want_exp=True), n * (4 + 1 + 4 / 32 + 1 / 32))
    res["cfg1_calculate_mx_qparam"] = timed(lambda: Q.calculate_mx_qparam(x, (-1,), 32, 127.0, True), n * (4 + 4 / 32))
    # the same ops on a 16x larger tensor (launch overhead amortised)
    xl = torch.randn(16384, 16384, generator=g, device=dev)
    nl = xl.numel()
    sl, cl = Q.quantize_mx(xl, q8, (-1,), 32, 127.0, True)
    res["large_quantize_mx_fp32_dropin_16384x16384"] = timed(lambda: Q.quantize_mx(xl, q8, (-1,), 32, 127.0, True), nl * (4 + 4 + 4 / 32), 5)
    res["large_dequantize_fp32_16384x16384"] = timed(lambda: Q.dequantize(cl, sl, None, (-1,), 32), nl * (4 + 4 + 4 / 32), 5)
    res["large_calculate_mx_qparam_16384x16384"] = timed(lambda: Q.calculate_mx_qparam(xl, (-1,), 32, 127.0, True), nl * (4 + 4 / 32), 5)
    res["large_quantize_mx_packed_int8_e8_16384x16384"] = timed(
        lambda: mq.quantize_tensors_mx([xl], q8, 32, 127.0, True, code_bits=8, want_exp=True), nl * (4 + 1 + 4 / 32 + 1 / 32), 5)
    xlb = xl.to(torch.bfloat16)
    res["large_quantize_mx_bf16_dropin_16384x16384"] = timed(lambda: Q.quantize_mx(xlb, q8, (-1,), 32, 127.0, True), nl * (2 + 2 + 2 / 32), 5)
    pk = mq.quantize_tensors_mx([xl], q8, 32, 127.0, True, code_bits=8, want_exp=True)[0]
    res["large_dequantize_packed_int8_e8_to_fp32_16384x16384"] = timed(
        lambda: mq.dequantize_packed(pk, torch.float32, use_exponent=True), nl * (1 + 1 / 32 + 4), 5)
    pk4 = mq.quantize_tensors_mx([xlb], tab("nf4"), 64, 1.0, code_bits=4)[0]
    res["large_dequantize_packed_nf4_to_bf16_16384x16384"] = timed(
        lambda: mq.dequantize_packed(pk4, torch.bfloat16), nl * (0.5 + 4 / 64 + 2), 5)
    del xl, sl, cl, xlb, pk, pk4
    vb.set_table_policy(allow_int=False)
    res["cfg1_quantize_mx_fp32_dropin_lut"] = timed(lambda: Q.quantize_mx(x, q8, (-1,), 32, 127.0, True), n * (4 + 4 + 4 / 32))
    vb.set_table_policy(allow_int=True)
    # cfg2: posit8_1 per-channel over ResNet-50-shaped conv weights (largest layer and a multi-tensor sweep)
    qp = tab("posit8_1")
    w = torch.randn(512, 512, 3, 3, generator=g, device=dev) * 0.02
    sc = w.abs().amax(dim=(1, 2, 3), keepdim=True) / 4096.0
    res["cfg2_quantize_posit8_perchannel_512x512x3x3"] = timed(lambda: Q.quantize(w, sc, None, None, None, qp), w.numel() * 8)
    wq = Q.quantize(w, sc, None, None, None, qp)
    res["cfg2_dequantize_perchannel_512x512x3x3"] = timed(lambda: Q.dequantize(wq, sc), w.numel() * 8)
    big = torch.randn(25_502_912 // 4608, 4608, generator=g, device=dev) * 0.02     # all 25.5 M weights as one tensor
    scb = big.abs().amax(dim=1, keepdim=True) / 4096.0
    res["cfg2_quantize_posit8_perchannel_25p5M"] = timed(lambda: Q.quantize(big, scb, None, None, None, qp), big.numel() * 8)
    # cfg4-shaped: fp32 [11008,4096] through a 16-entry codebook table, per-row scale
    w4 = torch.randn(11008, 4096, generator=g, device=dev) * 0.02
    cb = torch.from_numpy(vb.tables.codebook_table(sorted(torch.randn(16).mul(0.7).tolist())).view("int16").copy()).view(torch.bfloat16).to(dev)
    s4 = w4.abs().amax(dim=1, keepdim=True)
    res["cfg4_quantize_codebook16_perrow_11008x4096"] = timed(lambda: Q.quantize(w4, s4, None, None, None, cb), w4.numel() * 8)
    res["vmap_fp32_posit8_11008x4096"] = timed(lambda: Q.vmap(w4, qp), w4.numel() * 8)
    # cfg2 as one fused multi-tensor launch: all 54 ResNet-50 weight tensors, per-channel amax -> scale ->
    # posit8 code byte + dequantized fp32 (read 4N, write N + 4N)
    torch.manual_seed(1)
    rn = []
    for shp in resnet50_weight_shapes():
        t = torch.empty(shp, device=dev)
        torch.nn.init.kaiming_normal_(t, mode="fan_in")
        rn.append(t)
    n_rn = sum(t.numel() for t in rn)
    plan_a = mq.ChannelQuantPlan(rn, qp, 4096.0, want_codes=True, want_dequant=True)
    res["cfg2_fused_per_channel_posit8_54_tensors_25p5M"] = timed(plan_a.run, n_rn * 9)
    plan_b = mq.ChannelQuantPlan(rn, qp, 4096.0, want_values=True, want_dequant=False)
    res["cfg2_fused_per_channel_posit8_dropin_values_25p5M"] = timed(plan_b.run, n_rn * 8)
    del rn, plan_a, plan_b
    # cfg4: per-output-channel 16-entry quantile codebooks, W[11008,4096] fp32 ~ Student-t(5) * 0.02
    from voyager_compiler_b200 import codebook
    torch.manual_seed(3)
    wt = (torch.distributions.StudentT(5.0).sample((11008, 4096)) * 0.02).to(dev)
    lv = codebook.row_quantile_levels(wt, 16)
    res["cfg4_row_quantile_fit16_11008x4096"] = timed(lambda: codebook.row_quantile_levels(wt, 16), wt.numel() * 4 + lv.numel() * 4)
    qq = (2 * torch.arange(16, device=dev, dtype=torch.float32) + 1) / 32
    res["cfg4_torch_quantile_fit16_11008x4096_for_scale"] = timed(lambda: torch.quantile(wt, qq, dim=-1), wt.numel() * 4 + lv.numel() * 4)
    res["cfg4_row_codebook16_search_fp32_rule_11008x4096"] = timed(
        lambda: codebook.row_codebook_quantize(wt, lv, reference_rule=False), wt.numel() * 9 + lv.numel() * 4)
    res["cfg4_row_codebook16_search_reference_rule_11008x4096"] = timed(
        lambda: codebook.row_codebook_quantize(wt, lv, reference_rule=True), wt.numel() * 9 + lv.numel() * 4)
    res["cfg4_row_codebook16_indices_only_11008x4096"] = timed(
        lambda: codebook.row_codebook_quantize(wt, lv, reference_rule=False, want_values=False), wt.numel() * 5 + lv.numel() * 4)
    # statistics pass of the learned-codebook fit over the same weight: unit scale per block of 64, 4001 bins,
    # three fp64 moments, every element weighted by the energy of its input channel
    from voyager_compiler_b200 import lcq
    hist = lcq.Histogram(-7.0, 7.0)
    energy = torch.rand(4096, generator=g, device=dev) + 0.1
    res["lcq_accumulate_fp32_11008x4096_b64_energy"] = timed(lambda: hist.accumulate(wt, 64, 7.0, energy), wt.numel() * 4)
    res["lcq_accumulate_fp32_11008x4096_b64_flat"] = timed(lambda: hist.accumulate(wt, 64, 7.0, None), wt.numel() * 4)
    # the same statistics through torch's own operators on this GPU (upstream's formulation), for scale
    t_edges = torch.linspace(-7.5, 7.5, 4002, device=dev, dtype=torch.float32)
    t_m = [torch.zeros(4001, dtype=torch.float64, device=dev) for _ in range(3)]

    def torch_stats():
        flat = wt.reshape(-1, 64)
        v = (flat / (flat.abs().amax(-1, keepdim=True).clamp_min(1e-12) / 7.0)).reshape(-1)
        idx = (torch.bucketize(v, t_edges, right=True) - 1).clamp_(0, 4000)
        vd, wd = v.double(), energy.repeat(v.numel() // 4096).double()
        t_m[0].index_add_(0, idx, wd)
        t_m[1].index_add_(0, idx, wd * vd)
        t_m[2].index_add_(0, idx, wd * vd * vd)
    res["lcq_torch_operators_fp32_11008x4096_b64_energy_for_scale"] = timed(torch_stats, wt.numel() * 4, iters=3)
    del t_m, t_edges
    # observer + fake-quantize forward (calibration / QAT): activations [8192, 4096] bf16 and fp32
    from voyager_compiler_b200 import fake_quantize as fqm
    for dt, nm, es in ((torch.bfloat16, "bf16", 2), (torch.float32, "fp32", 4)):
        a = torch.randn(8192, 4096, generator=g, device=dev).to(dt)
        na = a.numel()
        sc = (a.abs().amax() / 127.0).float()
        res[f"fq_amax_per_tensor_{nm}_8192x4096"] = timed(lambda: fqm.amax(a), na * es)
        res[f"fq_amax_per_channel_last_{nm}_8192x4096"] = timed(lambda: fqm.amax(a, -1), na * es)
        res[f"fq_fake_quantize_int8_per_tensor_{nm}_8192x4096"] = timed(lambda: fqm.fake_quantize(a, sc, q8), na * 2 * es)
        res[f"fq_mx_fake_quantize_int8_block32_{nm}_8192x4096"] = timed(
            lambda: fqm.mx_fake_quantize(a, q8, -1, 32, 127.0, True), na * (2 * es + es / 32))
        mod = fqm.FusedAmaxObsFakeQuantize("int8", qscheme="per_tensor_symmetric", quant_max=127.0, amax_history_len=16,
                                           device=dev)
        res[f"fq_module_forward_int8_per_tensor_{nm}_8192x4096"] = timed(lambda: mod(a), na * 3 * es)
        # the observer's optional steps: exponent histogram (one read), outlier split (read + write) and merge (2 reads + write)
        hist = torch.zeros(254, device=dev)
        thr = torch.tensor([3.0], device=dev)
        res[f"fq_exponent_histogram_{nm}_8192x4096"] = timed(lambda: fqm.exponent_histogram(a, hist), na * es)
        res[f"fq_outlier_split_{nm}_8192x4096"] = timed(lambda: fqm.outlier_split(a, thr), na * 2 * es)
        inl, _ = fqm.outlier_split(a, thr)
        res[f"fq_outlier_merge_{nm}_8192x4096"] = timed(lambda: fqm.outlier_merge(a, inl, thr), na * 3 * es)
        mod2 = fqm.FusedAmaxObsFakeQuantize("int8", qscheme="per_tensor_symmetric", quant_max=127.0, amax_history_len=16,
                                            device=dev, record_histogram=True, outlier_threshold=3.0)
        res[f"fq_module_forward_histogram_outliers_{nm}_8192x4096"] = timed(lambda: mod2(a), na * 9 * es)
        # group-wise affine fake-quantize (uint4, blocks of 128 along the last axis): read + write, two numbers per block
        res[f"fq_group_affine_uint4_block128_{nm}_8192x4096"] = timed(
            lambda: fqm.group_affine_fake_quantize(a, -1, 128, 0.0, 15.0), na * (2 * es + 2 * es / 128))
        del a, mod, mod2, inl
    for k, v in res.items():
        v["frac_of_measured_hbm_peak"] = v["gbs"] / peaks["hbm_gbs"]
    print(json.dumps({"workload": "element-wise configs (cfg1, cfg2, cfg4 shapes)", "results": res, "peak_hbm_gbs": peaks["hbm_gbs"],
                      "peak_kind": kind, "timing_context": _timing_context(torch, flush, copy_bytes=4096 * 4096 * 8, read_bytes=4096 * 4096 * 4)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=32, help="fewer than 32: reduced model for profiler captures")
    ap.add_argument("--kernel-only", action="store_true", help="device-timed part only (profiler captures)")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only (skip the other configurations)")
    ap.add_argument("--workload", default="model", choices=["model", "linear", "linear_f32", "elementwise", "channel", "conv"],
                    help="model: NF4 whole-model quantization (headline); linear: the cfg5 MX linear")
    ap.add_argument("--only", default=None, help="--workload conv: run the cases whose name contains this text")
    ap.add_argument("--m", type=int, default=8192, help="rows of the activation for --workload linear")
    args = ap.parse_args()
    if args.workload == "linear":
        run_linear(args)
        return
    if args.workload == "elementwise":
        run_elementwise(args)
        return
    if args.workload == "channel":
        run_channel(args)
        return
    if args.workload == "conv":
        run_conv(args)
        return
    if args.workload == "linear_f32":
        run_linear_f32(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
