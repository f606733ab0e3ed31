#!/usr/bin/env python
"""Benchmark of the MoC sparse SwiGLU FFN hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--ffn-type moc|moc_gcp|moc_2_8|dense]

Workload (N = 1 and every rank of N > 1): one MoC FFN layer at the 1b-preset shape
(d=2048, d_ffn=5461, K=1024), bf16, X [8, 2048, 2048] = 16 384 tokens per GPU, forward +
backward with an upstream gradient; a "step" is one such pass. Weights ~N(0, 0.02) (same on all
ranks), X and dY ~N(0, 1) (per-rank seed): seeded synthetic data with the shapes and
distributions of the reference's single-layer training benchmark
(benchmarks/training/benchmark_training_latency.py:20-22, :112-124). With N > 1 the tokens are
sharded (each rank runs its own 16 384), weight gradients are averaged with NCCL, overlapped
with the rest of the backward pass; weak scaling.

Prints one JSON line (rank 0). `value`: tokens/s of the whole job with inputs resident in HBM,
CUDA-event timed, max over ranks. `e2e`: the same through the public module API with HOST
(pinned) inputs: every step copies X and dY to the device and Y and dX back. `roofline`: the
tcgen05 GEMM kernel (all dense contractions of the step), timed live with events recorded
between the kernels of the timed steps. `cpu_baseline` / `--impl reference`: the CPU oracle
(restatement of the reference's PyTorch path) on the host cores.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

D, D_FFN, K_SEL = 2048, 5461, 1024
TOKENS = 8 * 2048
METRIC = "moc_ffn_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"
CPU_SAMPLE_TOKENS = 1024


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ffn-type", default="moc", choices=["moc", "moc_gcp", "moc_2_8", "moc_post_silu_abs", "dense"],
                    help="dense = the dense SwiGLU comparison row of the same shape")
    ap.add_argument("--tokens", type=int, default=TOKENS, help="tokens per GPU (default: the configs[1] batch)")
    ap.add_argument("--dump-kernels", action="store_true", help="print per-launch durations of the last step")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--workload", default="ffn", choices=["ffn", "train_130m", "decode_1b", "memory", "decode_ffn"],
                    help="ffn: the headline single-layer benchmark (default). train_130m / decode_1b: the end-to-end "
                         "rows (whole LLaMA-style model around the FFN plugin, moc_b200.host), one JSON line each")
    ap.add_argument("--batch", type=int, default=1, help="decode_ffn: token rows per call")
    ap.add_argument("--decode-kind", default="global_moc", choices=["global_moc", "moc_2of8", "dense"],
                    help="decode_ffn: which decode row")
    ap.add_argument("--graph", action="store_true",
                    help="decode_ffn: time replays of one CUDA graph that holds one call per weight set")
    ap.add_argument("--weight-sets", type=int, default=4,
                    help="decode_ffn: distinct weight sets cycled through (4 x 67 MB: beyond the 126 MB L2)")
    ap.add_argument("--overlap", type=int, default=-1,
                    help="N>1: 1 = start the gradient all-reduce beside the dX GEMM, 0 = after the backward pass, "
                         "-1 (default) = beside the GEMM on 2 GPUs only: on 4 and 8 GPUs the overlapped collective "
                         "was faster in most runs (8 GPUs, 32 SMs reserved: 3.06-3.18 against 3.34 ms per step) but "
                         "single runs took 4-5 ms when its CTAs did not all fit the reserved SMs")
    ap.add_argument("--reserve-sms", type=int, default=-1,
                    help="N>1 with --overlap: SMs the dX GEMM leaves free (default: 8 for the own kernel - measured on "
                         "4 GPUs: 2.866 / 2.853 / 2.885 / 2.931 ms per step with 4 / 8 / 16 / 24 SMs - and 16 for NCCL)")
    ap.add_argument("--reduce", default="symm", choices=["symm", "nccl"],
                    help="N>1: symm = the library's own all-reduce kernel over symmetric NVLink memory, started beside "
                         "the dX GEMM (falls back to nccl, on every rank, if the symmetric allocation cannot be set "
                         "up); nccl = one NCCL all-reduce of the gradient bucket")
    ap.add_argument("--nccl-max-ctas", type=int, default=0, help="N>1: cap on the CTAs of an NCCL kernel (0: NCCL default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode FFN micro-benchmark (N=1 only)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the extra records of the JSON line (ffn_type variants, sustained loop, strong-scaling "
                         "split, the reference's own CUDA path on this GPU)")
    return ap.parse_args()


def workload_config(args, world):
    return {
        "workload": f"configs[1]: single MoC FFN layer fwd+bwd, 1b preset d={D} d_ffn={D_FFN} K={K_SEL}, "
                    f"X[8,2048,{D}] bf16, ffn_type={args.ffn_type}",
        "tokens_per_gpu": args.tokens,
        "global_tokens": args.tokens * world,
        # how the gradients are reduced (own NVLink kernel or NCCL, beside the dX GEMM or after it) is reported in the
        # line's "reduce" key: it can change at run time (fallback), and both arms must print the same config
        "parallelism": (f"token-sharded dp{world}, the three weight gradients averaged over NVLink once per step"
                        if world > 1 else "single GPU"),
        "l2": "inputs larger than L2: every step streams >600 MB of activations, weights and scratch "
              "(126 MB L2), no explicit flush",
    }


# ----------------------------------------------------------------------------------------------
# CPU oracle leg (cpu_baseline and --impl reference)
# ----------------------------------------------------------------------------------------------


REF_DIR = ROOT / "baseline" / "_ref"


def reference_package():
    """The unmodified reference package (installed by baseline/install_ref.py), or None."""
    if not (REF_DIR / "moc" / "ffn.py").exists():
        return None
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    try:
        import moc
        return moc
    except Exception:
        return None


def cpu_step_fn(ffn_type):
    """One fwd+bwd pass over a CPU_SAMPLE_TOKENS-token sample of the workload on the host cores. With the reference
    package installed: its own pure-PyTorch module (MoCSwiGLUFFN(mode=...), moc/ffn.py:124-259, :372-497; the factory
    path needs CUDA, moc/ffn.py:135-136), kind "reference"; otherwise the CPU oracle restatement, kind "port"."""
    import torch
    from oracle import moc_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    x, dy, wg, wu, wd = O.make_inputs(CPU_SAMPLE_TOKENS, D, D_FFN, torch.bfloat16, seed=1234)
    moc = reference_package()
    if moc is not None:
        from moc.ffn import MoCSwiGLUFFN, StandardSwiGLUFFN
        m = (StandardSwiGLUFFN(D, D_FFN) if ffn_type == "dense" else MoCSwiGLUFFN(D, D_FFN, K_SEL, mode=ffn_type))
        m = m.to(torch.bfloat16).train()
        with torch.no_grad():
            m.gate_proj.weight.copy_(wg)
            m.up_proj.weight.copy_(wu)
            m.down_proj.weight.copy_(wd)
        xs = x.clone().requires_grad_(True)

        def step():
            m.zero_grad(set_to_none=True)
            xs.grad = None
            m(xs).backward(dy)

        return step, torch.get_num_threads(), "reference"
    select = {"moc_2_8": "2of8", "moc_post_silu_abs": "post_silu_abs"}.get(ffn_type, "topk")

    def step():
        if ffn_type == "dense":
            O.dense_forward_backward(x, wg, wu, wd, dy)
            return
        fwd = O.moc_forward(x, wg, wu, wd, K_SEL, select=select)
        if ffn_type == "moc_gcp":
            O.moc_backward(dy, x, wg, wu, wd, fwd["idx"], fwd["g_sel"], fwd["u_sel"])
        else:
            O.moc_backward(dy, x, wg, wu, wd, fwd["idx"], fwd["g_sel"], fwd["u_sel"], fwd["s_sel"], fwd["z_sel"])

    return step, torch.get_num_threads(), "port"


def _cpu_what(kind):
    return ("the reference's own MoCSwiGLUFFN / StandardSwiGLUFFN modules (pure PyTorch path)" if kind == "reference"
            else "the CPU oracle (restatement of the reference's PyTorch path)")


def cpu_baseline(ffn_type, budget_s=12.0):
    step, threads, kind = cpu_step_fn(ffn_type)
    step()
    n, t0 = 0, time.perf_counter()
    while True:
        step()
        n += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s and n >= 2 or n >= 200:
            break
    return {
        "value": CPU_SAMPLE_TOKENS * n / dt,
        "unit": UNIT,
        "cores": threads,
        "kind": kind,
        "sample": f"{n} fwd+bwd passes of {_cpu_what(kind)} over {CPU_SAMPLE_TOKENS} tokens of the same shape (bf16), "
                  f"{dt:.1f} s",
    }


def run_reference(args, rank, world):
    if rank != 0:
        return
    step, threads, kind = cpu_step_fn(args.ffn_type)
    for _ in range(max(1, args.warmup)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = CPU_SAMPLE_TOKENS * args.steps / dt
    cfg = workload_config(args, world)
    sample = (f"each step = one fwd+bwd pass of {_cpu_what(kind)} over a {CPU_SAMPLE_TOKENS}-token sample of the "
              f"workload (bf16), {threads} host threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU leg
# ----------------------------------------------------------------------------------------------


class ClockSampler:
    """Samples nvidia-smi every 20 ms in the background; stop(t0, t1) keeps the samples whose
    timestamps fall inside the wall-clock window [t0, t1] (the timed region)."""

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self, t0, t1):
        import datetime

        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in out.strip().splitlines():
            f = [s.strip() for s in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[1]), float(f[2]), float(f[3]),
                             [n for n, v in zip(names, f[5:9]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if t0 <= r[0] <= t1]
        note = "samples inside the timed region"
        if not inside:       # region shorter than the sampling period: fall back to the busiest samples
            inside = sorted(rows, key=lambda r: -r[3])[:3]
            note = "timed region shorter than the sampling period: the 3 highest-power samples around it"
        sm = sorted(r[1] for r in inside)
        reasons = sorted({n for r in inside for n in r[4]})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max((r[2] for r in inside), default=None),
                "power_w_max": max((r[3] for r in inside), default=None), "samples": len(inside),
                "reasons": reasons, "note": note}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return d, "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def bench_decode(dev, peaks, layers=24, groups=20):
    """Decode FFN latency at the 1b shape (BASELINE config 3): batches of 1, 8, 64 rows, global MoC (K=1024),
    MoC 2:8 and dense. One CUDA graph holds `layers` FFN calls, each on its own weight set (24 x 89 MB, far
    beyond the 126 MB L2, so weights stream from HBM as in a 24-layer decode step); the graph is replayed
    `groups` times between two CUDA events. Reports microseconds per FFN call and per token, and the
    achieved HBM bandwidth on the algorithmic bytes of the call."""
    import torch

    from moc_b200 import _lib
    from moc_b200.inference import InferenceMoCSwiGLUFFN

    k2 = (D_FFN // 8) * 2 + min(2, D_FFN % 8)
    gen = torch.Generator(device=dev).manual_seed(0)

    def make(k, grouped):
        mods = []
        for _ in range(layers):
            m = InferenceMoCSwiGLUFFN(D, D_FFN, k, *((2, 8) if grouped else (None, None)))
            m = m.to(device=dev, dtype=torch.bfloat16)
            with torch.no_grad():
                for p in m.parameters():
                    p.copy_(torch.randn(p.shape, device=dev, generator=gen) * 0.02)
            m.freeze_for_compile()
            mods.append(m)
        return mods

    results = {}
    mods_global = make(K_SEL, False)
    mods_28 = make(k2, True)
    hbm = float(peaks.get("hbm_gbs", 6650.0))

    def graph_time(call, n_calls):
        """us per call of `call(i)` for i < n_calls captured into one CUDA graph."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(n_calls):
                call(i)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(n_calls):
                call(i)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(groups):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        del graph
        return 1e3 * e0.elapsed_time(e1) / (groups * n_calls)

    def row(us_call, nbytes, batch, **extra):
        r = {"us_per_call": us_call, "us_per_token": us_call / batch, "algorithmic_mb": nbytes / 1e6,
             "achieved_gbs": nbytes / (us_call * 1e-6) / 1e9, "hbm_frac": nbytes / (us_call * 1e-6) / 1e9 / hbm}
        r.update(extra)
        return r

    for mode, mods, label in (("auto", mods_global, "global_moc"), ("auto", mods_28, "moc_2of8"),
                              ("dense_baseline", mods_global, "dense")):
        for batch in (1, 8, 64):
            x = torch.randn(batch, D, device=dev, dtype=torch.bfloat16, generator=gen)
            us_call = graph_time(lambda i: mods[i](x, mode=mode), layers)
            if label == "dense":
                nbytes, distinct = 3 * D_FFN * D * 2, D_FFN
            else:
                # gate fully streamed; W_up and W_down^T rows of the channels that at least one row of the batch
                # selects (counted on the first weight set with the masked reference's selection)
                with torch.no_grad():
                    _, idx = mods[0]._select_channels(mods[0].gate_proj(x))
                distinct = int(torch.unique(idx).numel())
                nbytes = D_FFN * D * 2 + 2 * distinct * D * 2
            results[f"{label}_b{batch}"] = row(us_call, nbytes, batch, distinct_rows=distinct)
    # L2-resident comparison (one weight set replayed back to back), the protocol of the reference's published
    # decode table (benchmarks/inference/benchmark_ffn_latency.py:180-195)
    x1 = torch.randn(1, D, device=dev, dtype=torch.bfloat16, generator=gen)
    for mode, mods, label in (("auto", mods_global, "global_moc"), ("auto", mods_28, "moc_2of8"),
                              ("dense_baseline", mods_global, "dense")):
        results[f"{label}_b1_l2_hot"] = {"us_per_call": graph_time(lambda i: mods[0](x1, mode=mode), layers)}

    # ---- the selected projections alone (north-star row: gathered down projection against the HBM roofline) ----
    lib = _lib.lib()
    for batch in (1, 8):
        xg = torch.randn(batch, D, device=dev, dtype=torch.bfloat16, generator=gen)
        with torch.no_grad():
            vals, idx = mods_global[0]._select_channels(mods_global[0].gate_proj(xg))
            idx, order = idx.sort(dim=-1)
            vals = torch.gather(vals, -1, order)
        idx16 = idx.to(torch.int16).contiguous()
        distinct = int(torch.unique(idx).numel())
        z = torch.randn(batch, K_SEL, device=dev, dtype=torch.bfloat16, generator=gen)
        y = torch.empty(batch, D, device=dev, dtype=torch.bfloat16)
        zo = torch.empty(batch, K_SEL, device=dev, dtype=torch.bfloat16)
        nws = lib.moc_decode_workspace_bytes(batch, D, D_FFN)
        ws = torch.empty(nws, device=dev, dtype=torch.uint8)

        def down(i):
            m = mods_global[i]
            _lib.check(lib.moc_decode_selected_down(batch, K_SEL, D, D_FFN, z.data_ptr(), idx16.data_ptr(),
                                                    m._down_weight_t.data_ptr(), y.data_ptr(), ws.data_ptr(), nws,
                                                    _lib.stream_ptr(dev)), "moc_decode_selected_down")

        def up(i):
            m = mods_global[i]
            _lib.check(lib.moc_decode_selected_up(batch, K_SEL, D, D_FFN, xg.data_ptr(), vals.data_ptr(),
                                                  idx16.data_ptr(), m.up_proj.weight.data_ptr(), zo.data_ptr(),
                                                  _lib.stream_ptr(dev)), "moc_decode_selected_up")

        results[f"gathered_down_alone_b{batch}"] = row(graph_time(down, layers), distinct * D * 2, batch,
                                                       distinct_rows=distinct, launches_per_call=2)
        results[f"selected_up_alone_b{batch}"] = row(graph_time(up, layers), distinct * D * 2, batch,
                                                     distinct_rows=distinct, launches_per_call=1)
    results["protocol"] = (f"{layers} distinct weight sets per CUDA graph (HBM-resident, not L2), {groups} replays, "
                           "CUDA events; bytes = W_gate once + the W_up and W_down^T rows of the distinct selected "
                           "channels of the batch (dense: all three matrices). The *_alone rows time one entry point "
                           "per graph node chain: a call of 4-8 MB is one dependent DRAM round trip (about 1 us) plus "
                           "about 1 us of launch latency per kernel node, which bounds its roofline fraction; inside "
                           "the persistent launch the two gathers share one round trip")
    return results


def _fresh_module(ffn_type, dev):
    import torch

    import moc_b200

    gw = torch.Generator().manual_seed(0)
    m = moc_b200.build_ffn(D, D_FFN, ffn_type, k=K_SEL)
    with torch.no_grad():
        for p_ in m.parameters():
            p_.copy_(torch.randn(p_.shape, generator=gw) * 0.02)
    return m.to(device=dev, dtype=torch.bfloat16).train()


def _time_steps(fn, steps, warmup=3):
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def bench_variants(dev, x, dy, main_type):
    """ms per fwd+bwd step of the other ffn_types that BASELINE configs[1] names, same shape, weights and inputs
    (the reference benchmark runs dense and MoC side by side: benchmark_training_latency.py:107-139)."""
    out = {}
    for ffn_type in ("moc", "moc_gcp", "moc_2_8", "dense"):
        if ffn_type == main_type:
            continue
        m = _fresh_module(ffn_type, dev)

        def step():
            m.zero_grad(set_to_none=True)
            x.grad = None
            m(x).backward(dy)

        ms = _time_steps(step, 20)
        out[ffn_type] = {"ms_per_step": ms, "tokens_per_s": x.shape[0] * x.shape[1] / (ms * 1e-3)}
        del m
    return out


def bench_reference_gpu(dev, x, dy):
    """The reference's own CUDA path on this GPU, same shape and inputs: build_ffn(..., "moc") (Triton helper kernels
    + cuBLAS, moc/ffn.py:584-609) and its dense FFN, timed like its benchmark (10 warm-up, 30 iterations,
    benchmark_training_latency.py:25-36). If the Triton path fails in this environment the error is recorded and the
    pure-PyTorch mode="moc" runs on CUDA instead."""
    import torch

    moc = reference_package()
    if moc is None:
        return {"unavailable": "baseline/_ref is not installed (baseline/install_ref.py)"}
    out = {}
    gw = torch.Generator().manual_seed(0)
    weights = [torch.randn(shape, generator=gw) * 0.02 for shape in ((D_FFN, D), (D_FFN, D), (D, D_FFN))]

    def load(m):
        with torch.no_grad():
            m.gate_proj.weight.copy_(weights[0])
            m.up_proj.weight.copy_(weights[1])
            m.down_proj.weight.copy_(weights[2])
        return m.to(device=dev, dtype=torch.bfloat16).train()

    def timed(m):
        def step():
            m.zero_grad(set_to_none=True)
            x.grad = None
            m(x).backward(dy)
        ms = _time_steps(step, 30, warmup=10)
        return {"ms_per_step": ms, "tokens_per_s": x.shape[0] * x.shape[1] / (ms * 1e-3)}

    try:
        out["dense"] = dict(timed(load(moc.build_ffn(D, D_FFN, "dense"))), path="nn.Linear (cuBLAS) + autograd")
    except Exception as e:   # noqa: BLE001
        out["dense"] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
    try:
        out["moc"] = dict(timed(load(moc.build_ffn(D, D_FFN, "moc", k=K_SEL))), path="stock factory path: Triton helper kernels + cuBLAS")
    except Exception as e:   # noqa: BLE001
        err = f"{type(e).__name__}: {str(e)[:300]}"
        try:
            from moc.ffn import MoCSwiGLUFFN
            out["moc"] = dict(timed(load(MoCSwiGLUFFN(D, D_FFN, K_SEL, mode="moc"))),
                              path="pure PyTorch mode='moc' on CUDA (the Triton path failed)", triton_error=err)
        except Exception as e2:   # noqa: BLE001
            out["moc"] = {"error": err, "fallback_error": f"{type(e2).__name__}: {str(e2)[:300]}"}
    return out


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    import moc_b200
    from moc_b200 import _lib
    from moc_b200.dp import GradAllReducer

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        if args.nccl_max_ctas > 0:
            os.environ["NCCL_MAX_CTAS"] = str(args.nccl_max_ctas)
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.lib()   # raises if the CUDA library is missing

    tokens = args.tokens
    gw = torch.Generator().manual_seed(0)
    module = moc_b200.build_ffn(D, D_FFN, args.ffn_type, k=K_SEL)
    with torch.no_grad():
        for p in module.parameters():
            p.copy_(torch.randn(p.shape, generator=gw) * 0.02)
    module = module.to(device=dev, dtype=torch.bfloat16).train()
    gx = torch.Generator().manual_seed(1234 + rank)
    x_host = torch.randn(8, tokens // 8, D, generator=gx).bfloat16().pin_memory()
    dy_host = torch.randn(8, tokens // 8, D, generator=gx).bfloat16().pin_memory()
    x = x_host.to(dev).requires_grad_(True)
    dy = dy_host.to(dev)
    reducers = {"r": None}
    reduce_note = None
    if world > 1:
        from moc_b200.dp import SymmGradReducer
        if args.reserve_sms < 0:
            args.reserve_sms = 8 if args.reduce == "symm" else 16
        if args.reduce == "symm":
            # the own kernel has a fixed CTA count, so it always fits beside the dX GEMM: overlap at every N
            overlap = True if args.overlap < 0 else bool(args.overlap)
            reducers["r"] = SymmGradReducer(average=True, overlap=overlap, reserve_sms=args.reserve_sms)
            args.overlap = int(overlap)
        else:
            if args.overlap < 0:
                args.overlap = 1 if world == 2 else 0
            reducers["r"] = GradAllReducer(average=True, overlap=bool(args.overlap), reserve_sms=args.reserve_sms)

    def step(xin, dyin):
        module.zero_grad(set_to_none=True)
        xin.grad = None
        y = module(xin)
        if reducers["r"] is not None:
            with reducers["r"]:
                y.backward(dyin)
        else:
            y.backward(dyin)
        return y

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    moc_b200.set_status_checks(True)    # one checked step: raises if a device-side wait timed out
    if world > 1 and args.reduce == "symm":
        # the first step sets up the symmetric gradient buffers; if that fails on any rank, every rank goes back
        # to the NCCL all-reduce
        failed, why = 0, ""
        try:
            step(x, dy)
            reducers["r"].check()
        except Exception as exc:      # noqa: BLE001 - any set-up failure selects the fallback
            failed, why = 1, f"{type(exc).__name__}: {exc}"
        flag = torch.tensor([failed], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if int(flag.item()):
            reduce_note = "nccl (symmetric-memory reducer unavailable" + (f": {why[:200]}" if why else " on another rank") + ")"
            moc_b200.ffn.set_grad_ready_hook(None)
            moc_b200.ffn.set_bucket_provider(None)
            lib.moc_set_overlap_sm_reserve(0)
            args.reduce = "nccl"
            args.reserve_sms = 16
            args.overlap = 1 if world == 2 else 0
            reducers["r"] = GradAllReducer(average=True, overlap=bool(args.overlap), reserve_sms=args.reserve_sms)
            step(x, dy)
        else:
            reduce_note = ("own kernel over symmetric memory, " +
                           ("in-switch reduction (multimem)" if reducers["r"].multicast else "peer loads and stores") +
                           f", {reducers['r'].ctas} CTAs")
    else:
        step(x, dy)
    moc_b200.set_status_checks(False)
    dp_check = None
    if world > 1:
        # Gradient averaging, checked before anything is timed: with the SAME inputs on every rank the averaged
        # weight gradients must equal the local ones up to the rounding of the bf16 partial sums inside the
        # collective (exact on 2 ranks; 3 v, 5 v, ... need one more mantissa bit than v): relative L2 <= 2^-8.
        gs = torch.Generator().manual_seed(4321)
        xc = torch.randn(8, 64, D, generator=gs).bfloat16().to(dev).requires_grad_(True)
        dyc = torch.randn(8, 64, D, generator=gs).bfloat16().to(dev)
        module.zero_grad(set_to_none=True)
        module(xc).backward(dyc)
        torch.cuda.synchronize()
        local = [p_.grad.clone() for p_ in module.parameters()]
        step(xc, dyc)
        torch.cuda.synchronize()
        same = all(float((a_.float() - p_.grad.float()).norm() / a_.float().norm().clamp_min(1e-30)) <= 2.0 ** -8
                   for a_, p_ in zip(local, module.parameters()))
        flag = torch.tensor([1 if same else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        dp_check = "averaged weight gradients equal the local ones on every rank" if int(flag.item()) == 1 else "MISMATCH"
        if dp_check == "MISMATCH":
            raise RuntimeError("data-parallel check failed: averaged gradients differ from the local gradients")
    for _ in range(max(3, args.warmup)):
        step(x, dy)
    barrier()

    # ---- timed region: K steps, HBM-resident inputs, per-kernel events between launches ----
    cap = min(4096, 16 * args.steps + 16)
    prof_events = [torch.cuda.Event(enable_timing=True) for _ in range(cap)]
    for ev in prof_events:
        ev.record()    # forces creation of the underlying cudaEvent_t
    torch.cuda.synchronize()
    handles = (ctypes.c_void_p * cap)(*[ev.cuda_event for ev in prof_events])
    tags = (ctypes.c_int * cap)()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    side0 = lib.moc_side_launch_count()
    _lib.check(lib.moc_profile_begin(handles, cap), "moc_profile_begin")
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    epoch0 = time.time()
    t_start.record()
    for _ in range(args.steps):
        step(x, dy)
    t_end.record()
    torch.cuda.synchronize()
    n_prof = lib.moc_profile_end(tags, cap)
    side1 = lib.moc_side_launch_count()
    barrier()
    wall = time.perf_counter() - wall0
    clocks = sampler.stop(epoch0, epoch0 + wall) if rank == 0 else None
    ms_total = t_start.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())

    # per-kernel durations from the event profile
    kinds = {1: "gemm_tcgen05", 2: "gemm_simt", 3: "topk_select", 4: "select_2of8", 5: "expand_z", 6: "transpose",
             12: "bwd_sparse"}
    per_kind = {}
    launches = 0
    # every FFN call ends with a tag-0 event (forward and backward: two per step); only whole steps are evaluated,
    # so a profile that filled its event buffer before the last step still gives per-step figures
    n_rec = min(n_prof, cap)
    ends = [i for i in range(n_rec) if tags[i] == 0]
    steps_profiled = len(ends) // 2
    last = ends[2 * steps_profiled - 1] if steps_profiled else 0
    for i in range(last):
        tag = tags[i]
        if tag == 0:
            continue
        launches += 1
        dur = prof_events[i].elapsed_time(prof_events[i + 1])
        name = kinds.get(tag, f"tag{tag}")
        tot, cnt = per_kind.get(name, (0.0, 0))
        per_kind[name] = (tot + dur, cnt + 1)
    if steps_profiled and steps_profiled != args.steps:
        launches = round(launches * args.steps / steps_profiled)
    launches += side1 - side0     # tail-row GEMM launches on the side stream (no event)
    # the tensor-core GEMM launches of a step in launch order (side-stream tail launches carry no event)
    gemm_names = {"moc": ["gate+up", "down", "dZ", "dW (3 products)", "dX"],
                  "dense": ["gate", "up (+SwiGLU)", "down", "dZ", "dW (3 products)", "dX"]}
    names = gemm_names["dense" if args.ffn_type == "dense" else "moc"]
    gemm_rows = {}
    seq = 0
    for i in range(last):
        if tags[i] == 0:
            if i in ends[1::2]:
                seq = 0          # the backward call of a step has ended: next step
            continue
        if tags[i] == 1:
            nm = names[seq] if seq < len(names) else f"gemm{seq}"
            tot, cnt = gemm_rows.get(nm, (0.0, 0))
            gemm_rows[nm] = (tot + prof_events[i].elapsed_time(prof_events[i + 1]), cnt + 1)
            seq += 1
    flops_of = {"gate+up": 4.0, "gate": 2.0, "up (+SwiGLU)": 2.0, "down": 2.0, "dZ": 2.0, "dW (3 products)": 6.0, "dX": 4.0}
    peaks, peak_src = load_peaks()
    gemm_ms, gemm_n = per_kind.get("gemm_tcgen05", (0.0, 0))
    flops_per_step = 18.0 * tokens * D * D_FFN
    k_eff = K_SEL
    roofline = None
    if gemm_n:
        achieved = flops_per_step * steps_profiled / (gemm_ms * 1e-3) / 1e12
        peak_sust = float(peaks.get("bf16_tflops_sustained", 1400.0))
        peak_burst = float(peaks.get("bf16_tflops", 1590.0))
        # A timed region of well under a second runs at boost clocks without reaching the power cap: the burst
        # figure is the honest denominator there; a region of seconds settles under the cap: sustained figure.
        burst_region = ms_total < 1000.0
        peak = peak_burst if burst_region else peak_sust
        roofline = {
            "bound": "tensor", "kernel": "gemm_tcgen05_pair_kernel", "achieved": achieved, "peak": peak,
            "unit": "TFLOP/s", "frac": achieved / peak,
            "peak_source": f"{peak_src} ({'burst' if burst_region else 'sustained'} cuBLAS bf16; timed region "
                           f"{ms_total:.0f} ms)",
            "peak_burst": peak_burst, "frac_burst": achieved / peak_burst,
            "peak_sustained": peak_sust, "frac_sustained": achieved / peak_sust,
            "launches": gemm_n, "avg_launch_ms": gemm_ms / gemm_n,
            "algorithmic_flops_per_step": flops_per_step,
            # dram__bytes_read.sum + dram__bytes_write.sum per launch, mean over the five pair-kernel launches of a
            # step (2.98 GB per step; 2.22 GB algorithmic): copied from the ncu capture summarised in
            # profiles/gemm_tcgen05_pair_train_1b.md, not measured in this run
            "traffic": 0.596e9 if args.ffn_type in ("moc", "moc_gcp") else None,
            "traffic_source": "profiles/gemm_tcgen05_pair_train_1b.md (ncu capture of this workload)",
            "gemm_launches": {
                nm: {"ms": tot / cnt, "tflops": flops_of.get(nm, 0.0) * tokens * D * D_FFN / (tot / cnt * 1e-3) / 1e12,
                     "frac_of_burst_peak": flops_of.get(nm, 0.0) * tokens * D * D_FFN / (tot / cnt * 1e-3) / 1e12 / peak_burst}
                for nm, (tot, cnt) in gemm_rows.items() if cnt},
        }
    kernel_share = {name: {"ms_per_step": tot / max(1, steps_profiled), "launches_per_step": cnt / max(1, steps_profiled)}
                    for name, (tot, cnt) in sorted(per_kind.items())}
    if args.dump_kernels and rank == 0:
        # launch-by-launch durations of the last timed step, in launch order
        n = min(n_prof, cap)
        per_step = max(1, n // max(1, args.steps))
        seq = [(kinds.get(tags[i], "end"), round(prof_events[i].elapsed_time(prof_events[i + 1]), 4))
               for i in range(max(0, n - per_step), n - 1)]
        print("last step, launch order:", seq, file=sys.stderr, flush=True)

    # ---- e2e: host (pinned) inputs in, host outputs back, every step ----
    e2e = None
    if not args.no_e2e:
        # Software pipeline over steps, as an input pipeline would run it: the host->device copy of step i+1
        # and the device->host copy of step i-1 overlap the kernels of step i (two device buffer sets, one
        # copy stream per direction). Every copy of every step is inside the timed region.
        # empty_like does not inherit the pinned property; a pageable destination would make every result copy
        # synchronous and staged
        y_host = [torch.empty(x_host.shape, dtype=x_host.dtype, pin_memory=True) for _ in range(2)]
        dx_host = [torch.empty(x_host.shape, dtype=x_host.dtype, pin_memory=True) for _ in range(2)]
        assert x_host.is_pinned() and dy_host.is_pinned() and y_host[0].is_pinned() and dx_host[0].is_pinned()
        x_dev = [torch.empty_like(x).requires_grad_(True) for _ in range(2)]
        dy_dev = [torch.empty_like(dy) for _ in range(2)]
        in_ready = [torch.cuda.Event() for _ in range(2)]
        compute_done = [torch.cuda.Event() for _ in range(2)]
        s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()

        def h2d(i):
            j = i & 1
            with torch.cuda.stream(s_in), torch.no_grad():
                s_in.wait_event(compute_done[j])          # the kernels that last read this buffer set are done
                x_dev[j].copy_(x_host, non_blocking=True)
                dy_dev[j].copy_(dy_host, non_blocking=True)
                in_ready[j].record(s_in)

        def compute_and_d2h(i):
            j = i & 1
            s_main.wait_event(in_ready[j])
            y = step(x_dev[j], dy_dev[j])
            grad = x_dev[j].grad
            compute_done[j].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(compute_done[j])
                y_host[j].copy_(y.detach(), non_blocking=True)
                dx_host[j].copy_(grad, non_blocking=True)
                y.record_stream(s_out)
                grad.record_stream(s_out)

        def run_pipeline(n):
            h2d(0)
            for i in range(n):
                if i + 1 < n:
                    h2d(i + 1)
                compute_and_d2h(i)
            s_main.wait_stream(s_out)

        for ev in compute_done:
            ev.record(s_main)
        run_pipeline(3)
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        s_in.wait_event(e0)
        run_pipeline(args.steps)
        e1.record()
        torch.cuda.synchronize()
        barrier()
        e_ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms = float(t.item())
        nbytes = x_host.numel() * 2
        e2e = {"value": tokens * world * args.steps / (e_ms * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": 2 * nbytes, "d2h_bytes_per_step": 2 * nbytes,
               "ms_per_step": e_ms / args.steps,
               "what": "module(x).backward(dy) with x, dy copied from pinned host memory and y, dx copied back to "
                       "pinned host memory every step; copies of neighbouring steps overlap the kernels "
                       "(double-buffered, one copy stream per direction)"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(args.ffn_type)
    decode = None
    if rank == 0 and world == 1 and not args.no_decode:
        torch.cuda.empty_cache()
        decode = bench_decode(dev, peaks)

    # ---- extra records: strong-scaling split, sustained loop, ffn_type variants, the reference's CUDA path ----
    strong = sustained = variants = reference_gpu = None
    if not args.no_extras and world > 1 and tokens % (8 * world) == 0:
        # configs[1] read literally: the 16 384 tokens of ONE batch split over the ranks
        per = tokens // world
        xs = x.detach()[:, : per // 8].contiguous().requires_grad_(True)
        dys = dy[:, : per // 8].contiguous()
        for _ in range(3):
            step(xs, dys)
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            step(xs, dys)
        s1.record()
        torch.cuda.synchronize()
        barrier()
        t = torch.tensor([s0.elapsed_time(s1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        strong = {"tokens_per_gpu": per, "global_tokens": tokens, "ms_per_step": float(t.item()) / args.steps,
                  "tokens_per_s": tokens * args.steps / (float(t.item()) * 1e-3), "scaling": "strong"}
    if not args.no_extras and world == 1 and rank == 0:
        n_sus = max(args.steps, int(2200.0 / max(0.1, ms_total / args.steps)))
        sampler2 = ClockSampler(local_rank)
        sampler2.start()
        time.sleep(0.2)
        w0 = time.time()
        ms_sus = _time_steps(lambda: step(x, dy), n_sus, warmup=0)
        clocks_sus = sampler2.stop(w0, time.time())
        sustained = {"steps": n_sus, "ms_per_step": ms_sus, "tokens_per_s": tokens / (ms_sus * 1e-3),
                     "seconds": n_sus * ms_sus * 1e-3, "clocks": clocks_sus}
        variants = bench_variants(dev, x, dy, args.ffn_type)
        try:
            reference_gpu = bench_reference_gpu(dev, x, dy)
        except Exception as e:   # noqa: BLE001
            reference_gpu = {"error": f"{type(e).__name__}: {str(e)[:300]}"}

    if rank == 0:
        value = tokens * world * args.steps / (ms_total * 1e-3)
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args, world), "e2e": e2e, "gpu_launches": launches,
            "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks, "kernels": kernel_share,
            "host_wall_ms_per_step": 1e3 * wall / args.steps, "k_selected": k_eff, "decode": decode,
            "strong": strong, "sustained": sustained, "variants": variants, "reference_gpu": reference_gpu,
            "dp_check": dp_check,
            "reduce": ((reduce_note or "one NCCL all-reduce of the gradient bucket") +
                       (f", started beside the dX GEMM ({args.reserve_sms} SMs reserved)" if args.overlap else
                        ", after the backward pass")) if world > 1 else None,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_train_130m(args, rank, world, local_rank):
    """End-to-end training step of the 130m preset (d=768, d_ffn=2048, 12 layers, 12 heads, K=384, vocab 32100,
    64 x 256 tokens per GPU, synthetic ids with 10 % trailing pad labels, AdamW lr 2.5e-3): forward, loss, backward,
    optimizer step. Attention, norms, embedding, LM head and the optimizer are PyTorch ops; every FFN is this
    library's. Data parallel over ranks with DistributedDataParallel."""
    import torch
    import torch.distributed as dist

    from moc_b200 import host

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = host.get_config("130m", vocab_size=32100)
    torch.manual_seed(0)
    model = host.build_model(cfg, args.ffn_type).to(device=dev, dtype=torch.bfloat16)
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank]) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=2.5e-3, betas=(0.9, 0.999), weight_decay=0.0)
    batch, seq = 64, 256
    ids, labels = host.synthetic_batch(cfg, batch, seq, pad_fraction=0.1, seed=1234 + rank, device=dev)

    def step():
        opt.zero_grad(set_to_none=True)
        _, loss = net(ids, labels=labels)
        loss.backward()
        opt.step()
        return loss

    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        tokens = batch * seq * world * args.steps
        print(json.dumps({
            "metric": "e2e_130m_train_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "configs[3]: LLaMA-style 130m model training step, d=768 d_ffn=2048 12 layers 12 heads "
                                   f"K=384 vocab 32100, 64 x 256 tokens per GPU, AdamW, ffn_type={args.ffn_type}; host ops "
                                   "(attention, norms, LM head, optimizer) are PyTorch, FFNs are this library",
                       "parameters": model.num_parameters(), "final_loss": float(loss.item()),
                       "parallelism": f"DistributedDataParallel x{world}" if world > 1 else "single GPU"},
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_decode_1b(args, rank, world, local_rank):
    """End-to-end greedy decode of the 1b preset (d=2048, d_ffn=5461, 24 layers, 32 heads, K=1024, vocab 32100,
    bf16 weights and KV cache, 128 prompt tokens, 256 generated tokens) at batch 1 and 16, every decode step replayed
    from one CUDA graph. Single GPU."""
    import torch

    from moc_b200 import host

    if rank != 0:
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cfg = host.get_config("1b", vocab_size=32100, max_seq_len=384)
    torch.manual_seed(0)
    with torch.device(dev):
        model = host.build_model(cfg, args.ffn_type).to(dtype=torch.bfloat16).eval()
    results = {}
    for batch in (1, 16):
        prompt = torch.randint(0, cfg.vocab_size, (batch, 128), generator=torch.Generator().manual_seed(7)).to(dev)
        dec = host.GreedyDecoder(model, batch)
        dec.generate_graphed(prompt, 8)            # warm-up: allocations, first captures
        torch.cuda.synchronize()
        dec = host.GreedyDecoder(model, batch)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = dec.generate_graphed(prompt, 256)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        results[f"b{batch}"] = {"ms_total": ms, "ms_per_token": ms / 256, "tokens_per_s": batch * 256 / (ms * 1e-3),
                                "generated": list(out.shape)}
    print(json.dumps({
        "metric": "e2e_1b_decode_tokens_per_s", "value": results["b1"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
        "steps": 256, "warmup": 8, "ms_per_step": results["b1"]["ms_per_token"], "higher_is_better": True,
        "scaling": "replicas only", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "configs[4]: 1b model greedy decode, d=2048 d_ffn=5461 24 layers 32 heads K=1024 vocab "
                               f"32100, prompt 128, 256 new tokens, batch 1 and 16, ffn_type={args.ffn_type}; the timed "
                               "region includes the prompt pass, the graph capture and 255 graph replays",
                   "parameters": model.num_parameters()},
        "batches": results,
    }), flush=True)


def run_decode_ffn(args):
    """One decode row of BASELINE config 3 as plain stream launches (no CUDA graph): `--steps` calls of the decode
    FFN at `--batch` rows, cycling through `--weight-sets` distinct weight sets so that the weights come from HBM.
    A small case for profilers and for quick timing; the graph-replayed figures of the headline line come from
    bench_decode()."""
    import torch

    from moc_b200.inference import InferenceMoCSwiGLUFFN

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(0)
    grouped = args.decode_kind == "moc_2of8"
    k = (D_FFN // 8) * 2 + min(2, D_FFN % 8) if grouped else K_SEL
    mods = []
    for _ in range(args.weight_sets):
        m = InferenceMoCSwiGLUFFN(D, D_FFN, k, *((2, 8) if grouped else (None, None))).to(device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            for p in m.parameters():
                p.copy_(torch.randn(p.shape, device=dev, generator=gen) * 0.02)
        m.freeze_for_compile()
        mods.append(m)
    mode = "dense_baseline" if args.decode_kind == "dense" else "auto"
    x = torch.randn(args.batch, D, device=dev, dtype=torch.bfloat16, generator=gen)
    for i in range(args.warmup):
        mods[i % len(mods)](x, mode=mode)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        y = mods[i % len(mods)](x, mode=mode)
    e1.record()
    torch.cuda.synchronize()
    us = 1e3 * e0.elapsed_time(e1) / max(1, args.steps)
    out = {"workload": "decode_ffn", "kind": args.decode_kind, "batch": args.batch, "steps": args.steps,
           "warmup": args.warmup, "weight_sets": args.weight_sets, "us_per_call_stream_launches": us,
           "finite": bool(torch.isfinite(y.float()).all())}
    if args.graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for m in mods:
                m(x, mode=mode)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for m in mods:
                m(x, mode=mode)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        reps = max(1, args.steps // len(mods))
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        out["us_per_call_graph"] = 1e3 * e0.elapsed_time(e1) / (reps * len(mods))
    print(json.dumps(out))


def run_memory(args, rank, world, local_rank):
    """Peak training memory with the reference's protocol (benchmarks/memory/benchmark_memory.py:79-92: one warm-up
    step, reset_peak_memory_stats, one step, max_memory_allocated) for dense / moc / moc_gcp, on the 130m and 1b
    presets (batch 64 x 256, bf16 parameters, AdamW), plus, for one FFN layer at the benchmarked shape, the bytes the
    autograd node keeps between forward and backward (the compact saved set that is the method's point,
    moc/ffn.py:166-169, :417) and the peak of a layer's forward + backward."""
    import gc

    import torch

    from moc_b200 import host

    if rank != 0:
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    def cleanup():
        gc.collect()
        torch.cuda.synchronize(dev)
        torch.cuda.empty_cache()

    layer = {}
    for ffn_type in ("dense", "moc", "moc_gcp"):
        cleanup()
        m = _fresh_module(ffn_type, dev)
        x = torch.randn(TOKENS, D, device=dev, dtype=torch.bfloat16).requires_grad_(True)
        dy = torch.randn(TOKENS, D, device=dev, dtype=torch.bfloat16)
        m(x).backward(dy)                       # warm-up: workspaces, cached W_down^T
        m.zero_grad(set_to_none=True)
        x.grad = None
        cleanup()
        base = torch.cuda.memory_allocated(dev)
        torch.cuda.reset_peak_memory_stats(dev)
        y = m(x)
        torch.cuda.synchronize(dev)
        held = torch.cuda.memory_allocated(dev) - base - y.numel() * y.element_size()
        y.backward(dy)
        torch.cuda.synchronize(dev)
        peak = torch.cuda.max_memory_allocated(dev) - base
        layer[ffn_type] = {"saved_between_fwd_and_bwd_mb": held / 1e6, "peak_fwd_bwd_above_resident_mb": peak / 1e6}
        del m, x, dy, y
    models = {}
    for preset, lr in (("130m", 2.5e-3), ("1b", 6.0e-4)):
        cfg = host.get_config(preset, vocab_size=32100)
        ids, labels = host.synthetic_batch(cfg, 64, 256, pad_fraction=0.1, seed=1234, device=dev)
        for ffn_type in ("dense", "moc", "moc_gcp"):
            cleanup()
            torch.cuda.reset_peak_memory_stats(dev)
            torch.manual_seed(0)
            with torch.device(dev):
                model = host.build_model(cfg, ffn_type).to(dtype=torch.bfloat16)
            opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=(0.9, 0.999), weight_decay=0.0, fused=False)

            def one_step():
                _, loss = model(ids, labels=labels)
                loss.backward()
                opt.step()
                opt.zero_grad(set_to_none=True)

            one_step()
            torch.cuda.synchronize(dev)
            torch.cuda.reset_peak_memory_stats(dev)
            one_step()
            torch.cuda.synchronize(dev)
            models[f"{preset}.{ffn_type}"] = {"peak_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9,
                                              "reserved_memory_gb": torch.cuda.max_memory_reserved(dev) / 1e9,
                                              "parameters": model.num_parameters()}
            del model, opt
        del ids, labels
    cleanup()
    print(json.dumps({
        "metric": "peak_training_memory_gb", "value": models["1b.moc"]["peak_memory_gb"], "unit": "GB", "n_gpus": 1,
        "steps": 1, "warmup": 1, "ms_per_step": None, "higher_is_better": False, "scaling": "replicas only",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "peak training memory, reference protocol (one warm-up step, reset_peak_memory_stats, one "
                               "step, max_memory_allocated), batch 64 x 256, bf16 parameters, AdamW (not fused); host "
                               "model = moc_b200.host with this library's FFNs; value = 1b preset, ffn_type moc"},
        "models": models, "ffn_layer_16384_tokens": layer,
        "published_a800_1b_gb": {"dense": 60.54, "moc": 47.39, "moc_gcp": 45.78},
    }), flush=True)


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1:
        # launched without torchrun: re-exec under torch.distributed.run
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29531"),
               str(Path(__file__).resolve())] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload == "train_130m":
        run_train_130m(args, rank, world, local_rank)
        return
    if args.workload == "decode_1b":
        run_decode_1b(args, rank, world, local_rank)
        return
    if args.workload == "memory":
        run_memory(args, rank, world, local_rank)
        return
    if args.workload == "decode_ffn":
        run_decode_ffn(args)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
