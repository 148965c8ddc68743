#!/usr/bin/env python
"""Benchmark of the SLA attention hot path (forward + backward of SparseLinearAttention).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--impl ours|reference]

A step is one pass of the whole hot path over one batch of synthetic input: block-mask prediction,
fused sparse + linear forward, and the full backward, through the module API. One JSON line is
printed by rank 0. `value` is the dense-attention-equivalent TFLOP/s of the reference's own benchmark
formula (evaluate/bench_kernel.py:93-99: 4*B*H*L^2*D per forward, x3.5 for forward+backward), summed
over all ranks; ms per step, the sparse-actual TFLOP/s and the forward-only figures are extra keys.

N > 1: launched under torchrun, one rank per GPU, no collective on the attention path. Two splits are timed:
* `value` ("scaling": "weak"): rank r owns batch element r of a global batch of N, each batch element being the
  workload's B*H (batch, head) units, so per-GPU work is fixed;
* `strong`: the workload's own B*H units are sharded over the ranks (`sharding.unit_range`: c3 12 -> 6/3/{2,1},
  c5 16 -> 8/4/2, c4 40 -> 20/10/5), the total work is fixed. Per-unit checksums of o, dq, dk, dv of the sharded
  run are compared on rank 0 with those of the same units in its unsharded run: every unit must give the same
  bits however the units are split. `--gather` also times the optional NCCL all-gather of o.

--impl reference times the CPU restatement of the reference's algorithm (oracle/) on the host cores,
rank 0 only, each step a bounded sample (one head) of the same workload. That arm never imports the product
package or loads its shared library.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []
        self.t0 = self.t1 = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "10"], stdout=subprocess.PIPE, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, smax, reasons = [], None, set()
        inside = [ln for (ts, ln) in self.lines
                  if self.t0 is None or (self.t0 - 0.02 <= ts <= (self.t1 or ts) + 0.02)]
        if len(inside) < 3:          # very short region: fall back to everything sampled around it
            inside = [ln for (_, ln) in self.lines]
        for ln in inside:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def timed(fn, steps, warmup, sync):
    """W untimed warm-ups, then exactly `steps` calls between two events on the current stream."""
    for _ in range(warmup):
        fn()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    sync()
    return e0.elapsed_time(e1) / steps  # ms per call


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle restatement of the reference on host cores, on a bounded sample (one head)
# ------------------------------------------------------------------------------------------------
def cpu_reference_step(w, sample, backward=True):
    from oracle import sla_oracle as O
    q, k, v, do, W, b = sample
    t0 = time.perf_counter()
    _, lut, _ = O.get_block_map(q, k, w.topk, w.BLKQ, w.BLKK)   # on the given dtype (core.py:83)
    qf, kf, vf = (t.float().requires_grad_(backward) for t in (q, k, v))
    Wp, bp = W.clone().requires_grad_(backward), b.clone().requires_grad_(backward)
    o = O.sla_forward_gather_fp(qf, kf, vf, Wp, bp, lut, w.feature, w.BLKQ, w.BLKK)
    if backward:
        o.backward(do.float())
    return time.perf_counter() - t0


def load_synthetic():
    """The workload generator, loaded by file path: the CPU arm must not import the product package (whose
    __init__ loads libsla_b200.so)."""
    import importlib.util
    name = "sla_b200_synthetic_standalone"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "sla_b200", "synthetic.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def bench_config(w, world, impl="default", linear_scope="all"):
    """The `config` object both arms print (same keys, same values for the same command line)."""
    tensor_mb = w.B * w.H * w.L * w.D * 2 / 1e6
    return {"workload": w.name, "B_per_gpu": w.B, "H": w.H, "L": w.L, "D": w.D, "BLKQ": w.BLKQ, "BLKK": w.BLKK,
            "topk": w.topk, "topk_blocks": w.topk_blocks, "feature_map": w.feature,
            "global_units": world * w.units, "parallelism": f"bh-shard x{world}",
            "l2": "inputs larger than L2 (q,k,v,dO,o,dq,dk,dv = %.0f MB)" % (8 * tensor_mb), "impl": impl,
            "linear_scope": linear_scope}


def cpu_sample(w):
    synthetic = load_synthetic()
    q, k, v, do = synthetic.make_inputs(w, "cpu", units=[0])
    W, b = synthetic.make_proj(w, "cpu")
    return q, k, v, do, W, b


def _use_all_host_threads():
    """torchrun pins OMP_NUM_THREADS=1; the CPU arm is meant to use every core it may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def run_reference_arm(args, w, rank):
    if rank != 0:
        return
    cores = _use_all_host_threads()
    sample = cpu_sample(w)
    bwd = w.backward and not w.quantized
    for _ in range(args.warmup):
        cpu_reference_step(w, sample, bwd)
    ts = [cpu_reference_step(w, sample, bwd) for _ in range(args.steps)]
    sec = sum(ts) / len(ts)
    flops_unit = w.dense_equiv_flops(bwd) / w.units
    val = flops_unit / sec / 1e12
    what = "forward+backward" if bwd else "forward"
    line = {
        "impl": "reference", "metric": "sla_fwd_bwd_dense_equiv_tflops" if bwd else "sla_fwd_dense_equiv_tflops",
        "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(w, int(os.environ.get("WORLD_SIZE", "1"))),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"1 of {w.units} (batch,head) units, {what} incl. block map, per step"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# optional GPU baselines measured beside our arm (N = 1): reference Triton SLA, FlashAttention
# ------------------------------------------------------------------------------------------------
def load_reference_package():
    import importlib.util
    root = os.path.join(ROOT, "baseline", "_ref", "sparse_linear_attention")
    if not os.path.isdir(root):
        return None
    spec = importlib.util.spec_from_file_location("sla_reference", os.path.join(root, "__init__.py"),
                                                  submodule_search_locations=[root])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["sla_reference"] = mod
    spec.loader.exec_module(mod)
    return mod


def gpu_baselines(w, q, k, v, do, W, b, steps, warmup, backward=True):
    """Same box, same inputs: the unmodified reference module (Triton, bf16) and FlashAttention-2 dense.
    For the quantized workload both are forward-only 16-bit runs (the reference's own quantized module needs a
    package that is not installed)."""
    out = {}
    sync = torch.cuda.synchronize
    try:
        ref = load_reference_package()
        if ref is None:
            out["reference_triton"] = {"unavailable": "baseline/_ref not present"}
        else:
            BLKQ, BLKK = (128, 64) if w.quantized else (w.BLKQ, w.BLKK)
            m = ref.SparseLinearAttention(w.D, w.topk, w.feature, BLKQ, BLKK).cuda()
            with torch.no_grad():
                m.proj_l.weight.copy_(W)
                m.proj_l.bias.copy_(b)
            qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))

            def fwd():
                with torch.no_grad():
                    m(q, k, v)

            def fwdbwd():
                o = m(qg, kg, vg)
                o.backward(do)
                qg.grad = kg.grad = vg.grad = None

            f = timed(fwd, steps, warmup, sync)
            out["reference_triton"] = {"fwd_ms": f}
            if backward:
                fb = timed(fwdbwd, steps, warmup, sync)
                out["reference_triton"].update({"fwd_bwd_ms": fb,
                                                "fwd_bwd_dense_equiv_tflops": w.dense_equiv_flops(True) / fb / 1e9})
    except Exception as e:  # noqa: BLE001
        out["reference_triton"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    try:
        from flash_attn.flash_attn_interface import flash_attn_func
        qf, kf, vf = (t.transpose(1, 2).contiguous() for t in (q, k, v))
        dof = do.transpose(1, 2).contiguous() if backward else None
        if backward:
            qf, kf, vf = (t.requires_grad_(True) for t in (qf, kf, vf))

        def ffwd():
            with torch.no_grad():
                flash_attn_func(qf, kf, vf)

        def ffb():
            o = flash_attn_func(qf, kf, vf)
            o.backward(dof)
            qf.grad = kf.grad = vf.grad = None

        f = timed(ffwd, max(2, steps // 2), 2, sync)
        out["flash_attn_dense"] = {"fwd_ms": f, "fwd_tflops": w.dense_equiv_flops(False) / f / 1e9}
        if backward:
            fb = timed(ffb, max(2, steps // 2), 2, sync)
            out["flash_attn_dense"].update({"fwd_bwd_ms": fb, "fwd_bwd_tflops": w.dense_equiv_flops(True) / fb / 1e9})
    except Exception as e:  # noqa: BLE001
        out["flash_attn_dense"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    return out


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3")
    ap.add_argument("--no-baselines", action="store_true", help="skip the on-GPU reference/flash-attn timings")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--legacy-mma", action="store_true", help="force the mma.sync kernels")
    ap.add_argument("--graph", action="store_true",
                    help="also time the step replayed from CUDA graphs (sla_b200.graphed); reported as graph_ms_per_step")
    ap.add_argument("--single-stream", action="store_true",
                    help="keep every launch on one stream (the modules otherwise run the linear-branch state and "
                         "the quantization pre-passes on a second stream next to the block map)")
    ap.add_argument("--linear-scope", default="all", choices=["all", "unselected"],
                    help="scope of the linear branch: every token (the reference's code) or, per query block, the KV "
                         "blocks it did not select")
    ap.add_argument("--gather", action="store_true",
                    help="N > 1: also time the optional NCCL all-gather of the sharded run's output")
    ap.add_argument("--no-sustained", action="store_true", help="skip the 2 s sustained-clock loop (N = 1)")
    ap.add_argument("--topk", type=float, default=None, help="override the workload's top-k ratio (c5 sweeps 0.05/0.1/0.2)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        synthetic = load_synthetic()
        w = synthetic.WORKLOADS[args.workload]
        if args.topk is not None:
            w = dataclasses.replace(w, topk=args.topk)
        run_reference_arm(args, w, rank)
        return

    import torch.distributed as dist
    import sla_b200
    from sla_b200 import _lib, ops, sharding, synthetic
    w = synthetic.WORKLOADS[args.workload]
    if args.topk is not None:
        w = dataclasses.replace(w, topk=args.topk)

    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path for the product)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # rank r owns batch element r: units [r*units, (r+1)*units) of the global (batch x head) index
    unit_ids = [rank * w.units + u for u in range(w.units)]
    q, k, v, do = synthetic.make_inputs(w, dev, units=unit_ids)
    q, k, v, do = (t.view(w.B, w.H, w.L, w.D) for t in (q, k, v, do))
    W, b = synthetic.make_proj(w, dev)
    bwd = w.backward and not w.quantized
    if w.quantized:
        m = sla_b200.SageSparseLinearAttention(w.D, w.topk, w.feature).to(dev)
    else:
        m = sla_b200.SparseLinearAttention(w.D, w.topk, w.feature, w.BLKQ, w.BLKK,
                                           linear_scope=args.linear_scope).to(dev)
    if args.single_stream:
        m.overlap_linear_state = m.overlap_prepare = False   # default None: fork when the tensors are large enough
    with torch.no_grad():
        m.proj_l.weight.copy_(W)
        m.proj_l.bias.copy_(b)
    if args.legacy_mma and not w.quantized:
        m.impl_flags |= _lib.FLAG_LEGACY_MMA
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))

    def step_fwd():
        with torch.no_grad():
            return m(q, k, v)

    def step_fwdbwd():
        if not bwd:
            return step_fwd()
        o = m(qg, kg, vg)
        o.backward(do)
        qg.grad = kg.grad = vg.grad = None
        m.proj_l.weight.grad = m.proj_l.bias.grad = None

    # ---- main timed region: exactly K forward+backward steps ----
    sampler = ClockSampler(local_rank)
    sampler.start()
    def check_device(where):
        code = _lib.poll_device_error()
        if code:
            raise RuntimeError(f"device-side error {code} of a tcgen05 kernel during {where}: no number reported")

    for _ in range(args.warmup):
        step_fwdbwd()
    sync()
    check_device("warm-up")
    l0 = _lib.lib.sla_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark_begin()
    e0.record()
    for _ in range(args.steps):
        step_fwdbwd()
    e1.record()
    sync()
    sampler.mark_end()
    clocks = sampler.stop()
    launches = _lib.lib.sla_launch_count() - l0
    check_device("the timed region")
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    graph_ms = None
    if args.graph and bwd and not w.quantized:
        fast = sla_b200.graphed(m, qg, kg, vg)

        def step_graph():
            o = fast(qg, kg, vg)
            o.backward(do)
            qg.grad = kg.grad = vg.grad = None
            m.proj_l.weight.grad = m.proj_l.bias.grad = None

        graph_ms = timed(step_graph, args.steps, 3, sync)
        check_device("the graph replay")
    fwd_ms = timed(step_fwd, args.steps, 2, sync)
    if world > 1:
        t = torch.tensor([fwd_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        fwd_ms = float(t.item())

    # ---- sustained: the same step for at least 2 s, with the SM clock sampled over that loop (N = 1) ----
    sustained = None
    if world == 1 and not args.no_sustained:
        n_sus = max(args.steps, int(2200.0 / ms) + 1)
        s2 = ClockSampler(local_rank)
        s2.start()
        torch.cuda.synchronize()
        s2.mark_begin()
        sus_ms = timed(step_fwdbwd, n_sus, 0, torch.cuda.synchronize)
        s2.mark_end()
        c2 = s2.stop()
        check_device("the sustained loop")
        sustained = {"ms_per_step": sus_ms, "steps": n_sus, "seconds": sus_ms * n_sus / 1e3,
                     "value": w.dense_equiv_flops(bwd) / sus_ms / 1e9, "unit": "TFLOP/s", "clocks": c2}

    # ---- strong scaling: the workload's own B*H units sharded over the ranks ----
    def unit_checksums(ts):
        """Exact per-unit checksums (two int64 sums over the raw 16-bit patterns) of tensors shaped (1, U, L, D)."""
        out = []
        for t in ts:
            x = t.detach().reshape(t.shape[0] * t.shape[1], -1).view(torch.int16).to(torch.int64)
            wgt = (torch.arange(x.shape[1], device=x.device, dtype=torch.int64) % 8191) + 1
            out.append(torch.stack([x.sum(dim=1), (x * wgt).sum(dim=1)], dim=1))
        return torch.stack(out, dim=1)          # (U, n_tensors, 2)

    def run_units(mq, mk, mv, mdo):
        """One forward(+backward) step over the given units; returns the tensors whose bits are compared."""
        if not bwd:
            with torch.no_grad():
                return (m(mq, mk, mv),)
        a, b_, c = (t.detach().requires_grad_(True) for t in (mq, mk, mv))
        o = m(a, b_, c)
        o.backward(mdo)
        m.proj_l.weight.grad = m.proj_l.bias.grad = None
        return (o.detach(), a.grad, b_.grad, c.grad)

    strong = {"ms_per_step": ms, "units_per_rank": [w.units], "speedup": 1.0, "efficiency": 1.0,
              "granularity_bound": 1.0, "checksums_equal": None}
    if world > 1:
        counts = sharding.unit_counts(w.units, world)
        lo, hi = sharding.unit_range(w.units, rank, world)
        flat = lambda t: t.reshape(1, w.units, w.L, w.D)
        ref_sums = unit_checksums(run_units(*(flat(t) for t in (q, k, v, do)))) if rank == 0 else None
        if hi > lo:
            sq, sk, sv, sdo = synthetic.make_inputs(w, dev, units=list(range(lo, hi)))
            mine = run_units(sq, sk, sv, sdo)
            my_sums = unit_checksums(mine)
            strong_ms = timed(lambda: run_units(sq, sk, sv, sdo), args.steps, max(3, args.warmup), sync)
        else:                                   # more ranks than units: this rank idles through the same barriers
            mine, my_sums = None, torch.zeros((0, 4 if bwd else 1, 2), dtype=torch.int64, device=dev)
            strong_ms = timed(lambda: None, args.steps, max(3, args.warmup), sync)
        check_device("the sharded run")
        t = torch.tensor([strong_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        strong_ms = float(t.item())
        gathered = [None] * world
        dist.all_gather_object(gathered, my_sums.cpu())
        equal, mismatches = None, None
        if rank == 0:
            got = torch.cat(gathered, dim=0)
            equal = bool(torch.equal(got, ref_sums.cpu()))
            if not equal:       # which (unit, tensor) pairs differ
                names = ("o", "dq", "dk", "dv")
                bad = (got != ref_sums.cpu()).any(dim=-1).nonzero().tolist()
                mismatches = [f"unit {u}: {names[t]}" for u, t in bad][:16]
        bound = w.units / max(counts)
        strong = {"ms_per_step": strong_ms, "units_per_rank": counts, "speedup": ms / strong_ms,
                  "efficiency": ms / strong_ms / world, "granularity_bound": bound,
                  "efficiency_vs_granularity_bound": ms / strong_ms / bound,
                  "value": w.dense_equiv_flops(bwd) / strong_ms / 1e9, "unit": "TFLOP/s",
                  "checksums_equal": equal, "checksum_mismatches": mismatches,
                  "checksums": "per-unit int64 sums over the bits of " + ("o, dq, dk, dv" if bwd else "o") +
                               ", sharded run vs rank 0's unsharded run of the same units",
                  "baseline": "speedup = this run's replica ms_per_step (all units on every GPU) / sharded ms_per_step"}
        if args.gather:
            o_local = mine[0][0] if mine is not None else torch.zeros((0, w.L, w.D), dtype=q.dtype, device=dev)
            sharding.all_gather_units(o_local, w.units)
            g_ms = timed(lambda: sharding.all_gather_units(o_local, w.units), args.steps, 3, sync)
            t = torch.tensor([g_ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            strong["gather_ms"] = float(t.item())
            strong["gather_bytes_per_rank"] = w.units * w.L * w.D * 2
            # the forward as its own all-gather (sla_fwd_gather: the kernel's epilogue stores every output tile into the
            # peers' buffers as well) against forward + NCCL all-gather, forward only, same shards
            if hi > lo and min(counts) > 0:
                go = sharding.GatheredOutput(w.units, w.L, w.D, q.dtype, dev)

                def fwd_plain():
                    with torch.no_grad():
                        return m(sq, sk, sv)

                def fwd_nccl():
                    sharding.all_gather_units(fwd_plain()[0], w.units)

                def fwd_fused():
                    with torch.no_grad():
                        m(sq, sk, sv, gather=go)

                res = {}
                for name, fn in (("fwd_ms", fwd_plain), ("fwd_then_nccl_gather_ms", fwd_nccl),
                                 ("fwd_fused_gather_ms", fwd_fused)):
                    v_ms = timed(fn, args.steps, 3, sync)
                    t = torch.tensor([v_ms], dtype=torch.float64, device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    res[name] = float(t.item())
                go.full.zero_()
                sync()
                fwd_fused()
                go.wait()
                ref_full = sharding.all_gather_units(fwd_plain()[0], w.units)
                same = torch.tensor([1.0 if torch.equal(go.full, ref_full) else 0.0], device=dev)
                dist.all_reduce(same, op=dist.ReduceOp.MIN)
                res["fused_equals_nccl_on_every_rank"] = bool(same.item() == 1.0)
                strong["fused_gather"] = res
                check_device("the fused gather")
                del go
        del mine

    # ---- end to end through the module API with HOST buffers ----
    hq, hk, hv, hdo = (t.cpu().pin_memory() for t in (q, k, v, do))
    ho, hdq, hdk, hdv = (torch.empty_like(hq).pin_memory() for _ in range(4))

    # Steps are pipelined over three streams: while step i computes, the inputs of step i+1 come in and the
    # results of step i-1 go out (PCIe is full duplex). Every step still copies all of its inputs from pinned
    # host memory and all of its results back; device buffers are double-buffered.
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    n_in = 4 if bwd else 3
    dev_in = [[torch.empty_like(q) for _ in range(n_in)] for _ in range(2)]
    hosts_in = (hq, hk, hv, hdo)[:n_in]
    hosts_out = (ho, hdq, hdk, hdv) if bwd else (ho,)

    def e2e_run(steps):
        ev_in, ev_comp = [None, None], [None, None]

        def load(i):
            b = i & 1
            with torch.cuda.stream(s_in):
                if ev_comp[b] is not None:
                    s_in.wait_event(ev_comp[b])          # step i-2 has finished reading this buffer
                for d, h in zip(dev_in[b], hosts_in):
                    d.copy_(h, non_blocking=True)
                ev_in[b] = s_in.record_event()

        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        load(0)
        for i in range(steps):
            b = i & 1
            if i + 1 < steps:
                load(i + 1)
            cur.wait_event(ev_in[b])
            if bwd:
                dq_, dk_, dv_ = (t.detach().requires_grad_(True) for t in dev_in[b][:3])
                o = m(dq_, dk_, dv_)
                o.backward(dev_in[b][3])
                outs = (o.detach(), dq_.grad, dk_.grad, dv_.grad)
                m.proj_l.weight.grad = m.proj_l.bias.grad = None
            else:
                with torch.no_grad():
                    outs = (m(*dev_in[b]),)
            ev_comp[b] = cur.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp[b])
                for h, d in zip(hosts_out, outs):
                    h.copy_(d, non_blocking=True)
                    d.record_stream(s_out)
        cur.wait_stream(s_out)
        cur.wait_stream(s_in)

    e2e_steps = max(3, min(args.steps, 10))
    e2e_run(2)
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    sync()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    check_device("the end-to-end run")
    if world > 1:
        t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    tensor_bytes = q.numel() * q.element_size()

    # ---- the dominant kernels timed alone (CUDA events on the launching stream) ----
    peaks = _peaks()
    import ctypes as C
    BLKQ, BLKK = (128, 64) if w.quantized else (w.BLKQ, w.BLKK)
    bm = ops.block_map(q, k, w.topk, BLKQ, BLKK, want_cols=True)
    flags = _lib.FLAG_SPARSE_ONLY | (_lib.FLAG_LEGACY_MMA if args.legacy_mma else 0)
    shape = ops.make_shape(w.B, w.H, w.L, w.D, BLKQ, BLKK, bm.topk, torch.bfloat16, w.feature, flags=flags)
    o_s = torch.empty_like(q)
    lse = torch.empty((w.B, w.H, w.L), dtype=torch.float32, device=dev)
    st = torch.cuda.current_stream().cuda_stream

    Wz = torch.zeros(w.D, w.D, device=dev)

    def k_fwd():
        if w.quantized:   # quantization pre-passes + the 8-bit kernel (sparse branch only)
            ops.sage_sla_attention(q, k, v, Wz, None, bm, w.feature, sparse_only=True)
            return
        _lib.check(_lib.lib.sla_sparse_fwd(C.byref(shape), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                           bm.lut.data_ptr(), o_s.data_ptr(), lse.data_ptr(), st))

    dq_, dk_, dv_ = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    bws = ops._workspace(shape, _lib.OP_SPARSE_BWD, dev)

    def k_bwd():
        _lib.check(_lib.lib.sla_sparse_bwd(C.byref(shape), q.data_ptr(), k.data_ptr(), v.data_ptr(), o_s.data_ptr(),
                                           lse.data_ptr(), do.data_ptr(), bm.lut.data_ptr(),
                                           bm.col_offsets.data_ptr(), bm.col_index.data_ptr(), dq_.data_ptr(),
                                           dk_.data_ptr(), dv_.data_ptr(), bws.data_ptr(), bws.numel(), st))

    def k_map():
        ops.block_map(q, k, w.topk, BLKQ, BLKK, want_cols=True)

    # the fused front end (per-head RMS norm + rotary embedding + block sums) and the mask prediction from its sums
    front = {}
    if True:
        gain = torch.ones(w.D, device=dev)
        pos = torch.arange(w.L, device=dev, dtype=torch.float32)[:, None]
        inv = 10000.0 ** (-torch.arange(w.D // 2, device=dev, dtype=torch.float32) / (w.D // 2))
        rc, rs = torch.cos(pos * inv), torch.sin(pos * inv)
        q_f, k_f = torch.empty_like(q), torch.empty_like(k)
        holder = {}

        def k_front():
            holder["p"] = ops.qk_norm_rope_pool(q, k, gain, gain, rc, rs, 1e-6, True, BLKQ, BLKK)[2]

        def k_map_pooled():
            ops.block_map_pooled(holder["p"], w.topk, want_cols=True)

        fr_ms = timed(k_front, args.steps, 3, torch.cuda.synchronize)
        mp_ms = timed(k_map_pooled, args.steps, 3, torch.cuda.synchronize)
        front = {"qk_norm_rope_pool": {"ms": fr_ms, "gbs": 4 * tensor_bytes / fr_ms / 1e6},
                 "block_map_from_sums": {"ms": mp_ms}}
        del q_f, k_f, holder

    kf_ms = timed(k_fwd, args.steps, 3, torch.cuda.synchronize)
    if bwd:
        k_fwd()
    kb_ms = timed(k_bwd, args.steps, 3, torch.cuda.synchronize) if bwd else 0.0
    km_ms = timed(k_map, args.steps, 3, torch.cuda.synchronize)
    fwd_flops = w.sparse_flops(False)
    bwd_flops = w.sparse_flops(True) - fwd_flops
    kernels = {
        "sparse_fwd": {"ms": kf_ms, "tflops": fwd_flops / kf_ms / 1e9},
        "block_map": {"ms": km_ms, "gbs": 2 * tensor_bytes / km_ms / 1e6},
    }
    kernels.update(front)
    if bwd:
        kernels["sparse_bwd_dq_dkdv"] = {"ms": kb_ms, "tflops": bwd_flops / kb_ms / 1e9}
    # DRAM bytes per launch from the committed ncu captures (profiles/tcgen05_sparse_kernels_c3.md,
    # profiles/sage_fwd_tc_c4s.md): dram__bytes_read.sum + dram__bytes_write.sum; null where not captured.
    # The captures are the launches of a whole module step: the forward there also writes o (100 MB at c3) and
    # the dK/dV kernel also reads dH; the c4 figure is the 8-head capture times 5 (traffic grows with the heads).
    # The dQ figure is that capture's 592.7 MB plus what the kernel reads and writes since it also takes the row
    # statistics (o_s once, the statistics array): +18.9 MB in the 2-head capture of
    # profiles/tcgen05_sparse_kernels_c3s.md, times 6 for the 12 heads.
    traffic_table = {("c3", "sparse_fwd"): 471.8e6, ("c3", "sparse_bwd_dq_dkdv"): (592.7e6 + 6 * 18.9e6) + 585.9e6,
                     ("c4", "sparse_fwd"): 5 * 525.5e6, ("c4s", "sparse_fwd"): 525.5e6}
    if w.quantized:
        # no driver-measured 8-bit peak exists: measure an e4m3 GEMM here with the protocol of the bf16 one
        # (8192^3, best of 10, CUDA events) and quote it beside the bf16 peak
        try:
            n = 8192
            a8 = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
            b8 = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
            one = torch.ones((), device=dev)
            mm = lambda: torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            best = min(timed(mm, 1, 1, sync) for _ in range(10))
            peaks["e4m3_tflops"] = 2.0 * n ** 3 / best / 1e9
            del a8, b8
        except Exception as e:  # noqa: BLE001
            peaks["e4m3_tflops"] = None
            print(f"# e4m3 peak not measured: {type(e).__name__}: {e}"[:200], file=sys.stderr)
        try:        # the INT8 half of the kernel's GEMM work: s8 x s8 -> s32, same size and protocol
            n = 8192
            ai = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8)
            bi = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8).t()
            mmi = lambda: torch._int_mm(ai, bi)
            best = min(timed(mmi, 1, 1, sync) for _ in range(10))
            peaks["int8_tops"] = 2.0 * n ** 3 / best / 1e9
            del ai, bi
        except Exception as e:  # noqa: BLE001
            peaks["int8_tops"] = None
            print(f"# int8 peak not measured: {type(e).__name__}: {e}"[:200], file=sys.stderr)
    dom = "sparse_bwd_dq_dkdv" if kb_ms >= kf_ms else "sparse_fwd"
    achieved = kernels[dom]["tflops"]
    roofline = {"kernel": dom, "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                "traffic": traffic_table.get((w.name, dom)),
                "peak_source": peaks["source"] + " burst (kernel timed alone)",
                "algorithmic_flops_per_launch": bwd_flops if dom != "sparse_fwd" else fwd_flops}
    if w.quantized:
        # half of the kernel's GEMM work is INT8 (S = Q K^T), half e4m3 (P V): the denominator is the rate at which a
        # kernel doing both halves at their library-GEMM peaks would run (harmonic mean of the two measured peaks)
        e4, i8 = peaks.get("e4m3_tflops"), peaks.get("int8_tops")
        roofline["peak_e4m3_tflops_measured_here"] = e4
        roofline["peak_int8_tops_measured_here"] = i8
        roofline["frac_of_bf16_peak"] = roofline["frac"]
        if e4 and i8:
            p8 = 2.0 / (1.0 / e4 + 1.0 / i8)
            roofline.update({"peak": p8, "frac": achieved / p8,
                             "peak_source": "harmonic mean of the e4m3 and INT8 GEMM peaks measured in this run "
                                            "(torch._scaled_mm / torch._int_mm, 8192^3, best of 10)"})
        roofline["note"] = ("half of this kernel's GEMM work runs as INT8, half as e4m3; the kernel is bound by the "
                            "SFU (ex2) rate, not by the tensor pipe")

    dense_fb = w.dense_equiv_flops(bwd)
    value = world * dense_fb / ms / 1e9
    line = {
        "metric": "sla_fwd_bwd_dense_equiv_tflops" if bwd else "sla_fwd_dense_equiv_tflops", "value": value,
        "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8/e4m3" if w.quantized else "bf16", "data": "synthetic",
        "config": bench_config(w, world, "mma.sync" if args.legacy_mma else "default", args.linear_scope),
        "fwd_ms": fwd_ms, "fwd_bwd_ms": ms,
        "fwd_dense_equiv_tflops": world * w.dense_equiv_flops(False) / fwd_ms / 1e9,
        "sparse_actual_tflops": world * (w.sparse_flops(bwd) + w.linear_flops(bwd)) / ms / 1e9,
        "graph_ms_per_step": graph_ms,
        "mask_ms": kernels["block_map"]["ms"], "fwd_ms_excluding_mask": fwd_ms - kernels["block_map"]["ms"],
        "fwd_bwd_ms_excluding_mask": ms - kernels["block_map"]["ms"],
        "e2e": {"value": world * dense_fb / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "overlap": "steps pipelined over 3 streams (copy-in, compute, copy-out), 2 device buffers",
                "h2d_bytes_per_step": (4 if bwd else 3) * tensor_bytes,
                "d2h_bytes_per_step": (4 if bwd else 1) * tensor_bytes},
        "gpu_launches": int(launches), "clocks": clocks, "kernels": kernels, "roofline": roofline,
        "strong": strong, "sustained": sustained,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        _use_all_host_threads()
        sample = cpu_sample(w)
        cpu_reference_step(w, sample, bwd)
        ts, t_end = [], time.perf_counter() + 15.0
        while len(ts) < 2 or (time.perf_counter() < t_end and len(ts) < 8):
            ts.append(cpu_reference_step(w, sample, bwd))
        sec = sum(ts) / len(ts)
        line["cpu_baseline"] = {"value": dense_fb / w.units / sec / 1e12, "unit": "TFLOP/s",
                                "cores": torch.get_num_threads(), "kind": "port",
                                "sample": f"1 of {w.units} (batch,head) units x {len(ts)} repeats, "
                                          f"forward+backward incl. block map ({sec:.2f} s each)"}
    if rank == 0 and world == 1 and not args.no_baselines:
        line["gpu_baselines"] = gpu_baselines(w, q, k, v, do, W, b, max(3, min(10, args.steps // 2)), 3, backward=bwd)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
