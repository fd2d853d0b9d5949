#!/usr/bin/env python
"""Benchmark of the sparse-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload IDX] [--impl ours|reference]

A step is one full call of `spas_sage2_attn_meansim_topk_cuda(q, k, v, topk)` (predictor, INT8/FP8
quantisers, block-sparse attention) on one batch of synthetic inputs of the named workload.
Prints ONE JSON line (rank 0).  Metric: dense-equivalent TOPS = 4*B*H*N^2*D / time (causal: half).
With N GPUs every rank processes its own copy of the workload's heads (weak scaling, no collective
on the data path); the value is the sum over ranks divided by the slowest rank's time.

`--impl reference` times the CPU restatement of the reference algorithm (the reference has no CPU
implementation of its own and its CUDA extension cannot be built here) on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "dense_equivalent_attention_throughput_topk0.5"
PVTHRESHD = 50.0
UNIT = "TOPS"
NOMINAL_8BIT_TOPS = 4500.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", type=int, default=2, help="index into spargeattn_b200.synthetic.WORKLOADS")
    ap.add_argument("--topk", type=float, default=None)
    ap.add_argument("--pvthreshd", type=float, default=50.0, help="PV-skip threshold passed to the API (default 50)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-heads-per-chunk", type=int, default=2)
    ap.add_argument("--ulysses-heads-per-step", type=int, default=None,
                    help="workload 4 on several GPUs: heads per pipelined exchange/compute step")
    ap.add_argument("--quick", action="store_true", help="device-resident arm only (for profiler runs)")
    return ap.parse_args()


def workload_shape(w):
    if w["kind"] == "llm":
        n = w["N"]
    else:
        t, hh, ww = w["grid"]
        n = t * hh * ww + w.get("text", 0)
    return w["B"], w["H"], n, w["D"]


def dense_equiv_ops(B, H, N, D, causal):
    ops = 4.0 * B * H * float(N) * float(N) * D
    return ops / 2 if causal else ops


def config_dict(idx, w, topk, n_gpus, ulysses=False):
    B, H, N, D = workload_shape(w)
    sharding = (f"Ulysses sequence parallel over {n_gpus} GPUs: N/{n_gpus} tokens per rank, exchanged to "
                f"{H // n_gpus} full-length heads per rank and back ("
                f"{'pipelined copy-engine peer transfers' if n_gpus == 2 else 'NCCL all-to-all'}; strong scaling)") if ulysses else \
        f"{n_gpus} x full head set (weak scaling, no collective)"
    return {"workload": f"cfg{idx}:{w['name']} B={B} H={H} N={N} D={D} bf16 {'causal' if w['causal'] else 'non-causal'} "
                        f"topk={topk} pvthreshd={PVTHRESHD:g}",
            "per_gpu_heads": H // n_gpus if ulysses else H, "sharding": sharding,
            "l2_policy": "inputs larger than L2 (q,k,v = %.0f MB per rank)" % (3 * B * H * N * D * 2 / 1e6)}


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.samples, self.stop, self.th = index, [], threading.Event(), None

    def _run(self):
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self.stop.wait(0.05)

    def __enter__(self):
        self.th = threading.Thread(target=self._run, daemon=True)
        self.th.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.th.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(float(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": float(self.samples[0][1]), "reasons": reasons,
                "samples": len(mhz)}


# ------------------------------------------------------------------------------------------ CPU arm
_cpu_inputs = {}


def cpu_reference_sample(idx, w, topk, q_blocks):
    """Times the CPU restatement on one head: full preprocessing + attention on the first `q_blocks`
    query blocks, and extrapolates linearly in heads x query blocks.  Returns (tops, seconds, note)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import sparge_oracle as O
    from spargeattn_b200 import synthetic
    torch.set_num_threads(os.cpu_count())
    B, H, N, D = workload_shape(w)
    if idx not in _cpu_inputs:
        q, k, v = synthetic.workload_qkv(idx, "cpu", heads=1)
        _cpu_inputs[idx] = (q[:1], k[:1], v[:1])
    q, k, v = _cpu_inputs[idx]
    nq = (N + 127) // 128
    qb = min(q_blocks, nq)
    t0 = time.perf_counter()
    km = O.k_mean(k)
    pr = O.predictor(q, k, km, w["causal"], -0.1, None, topk, False)
    v8, vs = O.quant_v(v)
    t1 = time.perf_counter()
    rows = min(qb * 128, N)
    O.attention_dense_masked(pr["q_int8"][:, :, :rows], pr["q_scale"][:, :, :qb], pr["k_int8"], pr["k_scale"], v8, vs,
                             pr["map"][:, :, :qb], D ** -0.5, False, torch.bfloat16, q_chunk=512)
    t2 = time.perf_counter()
    full = (t1 - t0) * B * H + (t2 - t1) * B * H * nq / qb
    tops = dense_equiv_ops(B, H, N, D, w["causal"]) / full / 1e12
    note = (f"1 of {B * H} heads: full predictor+quantisers ({t1 - t0:.2f}s) + masked fp32 attention on the first {qb} "
            f"of {nq} query blocks ({t2 - t1:.2f}s); extrapolated linearly to all heads and blocks")
    return tops, full, (t2 - t0), note


def run_reference(args, idx, w, topk):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals, sample_s, note = [], 0.0, ""
    for i in range(args.warmup + args.steps):
        tops, full, sample_s, note = cpu_reference_sample(idx, w, topk, q_blocks=32)
        if i >= args.warmup:
            vals.append((tops, full))
    tops = sum(v[0] for v in vals) / len(vals)
    full = sum(v[1] for v in vals) / len(vals)
    line = {"impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": full * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8-qk/fp8-pv (emulated in fp32 on CPU)", "data": "synthetic",
            "config": config_dict(idx, w, topk, args.gpus),
            "cpu_baseline": {"value": tops, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": note},
            "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------ GPU arm
def main():
    global PVTHRESHD
    args = parse()
    PVTHRESHD = args.pvthreshd
    from spargeattn_b200 import synthetic
    idx = args.workload
    w = synthetic.WORKLOADS[idx]
    topk = args.topk if args.topk is not None else w["topk"]
    if args.impl == "reference":
        run_reference(args, idx, w, topk)
        return

    import spargeattn_b200 as S
    from spargeattn_b200 import core, ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    B, H, N, D = workload_shape(w)
    causal = w["causal"]
    # workload 4 on several GPUs: Ulysses sequence parallelism (strong scaling, two all-to-alls per call);
    # every other case: each rank runs the full head set on its own data (weak scaling, no collective)
    ulysses = world > 1 and w.get("ulysses", False)
    calls_per_step = 1
    gen_seed_shift = 0 if ulysses else rank
    if w["kind"] == "llm":
        q, k, v = synthetic.llm_prefill_qkv(B, H, N, D, idx + 100 * gen_seed_shift, dev)
    else:
        q, k, v = synthetic.video_qkv(B, H, w["grid"], D, idx + 100 * gen_seed_shift, dev, w.get("text", 0),
                                      w.get("text_first", True))
    if ulysses:
        from spargeattn_b200.sharding import ulysses_attention
        assert N % world == 0 and H % world == 0
        n_loc = N // world
        q, k, v = (t[:, :, rank * n_loc:(rank + 1) * n_loc].contiguous() for t in (q, k, v))
        if world == 2:      # peer exchange: one attention call per group of heads
            from spargeattn_b200.sharding import auto_heads_per_step
            hstep = args.ulysses_heads_per_step or auto_heads_per_step(B, N, H // world, dev)
            calls_per_step = -(-(H // world) // hstep)
        api = lambda a, b, c: ulysses_attention(a, b, c, topk=topk, is_causal=causal, pvthreshd=args.pvthreshd,
                                                heads_per_step=args.ulysses_heads_per_step)
    else:
        api = lambda a, b, c: S.spas_sage2_attn_meansim_topk_cuda(a, b, c, topk=topk, is_causal=causal,
                                                                 pvthreshd=args.pvthreshd)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    # ---- device-resident arm
    for _ in range(args.warmup):
        o = api(q, k, v)
    clk = ClockSampler(local)
    clk.__enter__()
    ms_step = timed(lambda: api(q, k, v), args.steps)
    ops.check_device_status(dev)
    total_ops = dense_equiv_ops(B, H, N, D, causal) * (1 if ulysses else world)
    value = total_ops / (ms_step * 1e-3) / 1e12

    if args.quick:
        clk.__exit__()
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                              "warmup": args.warmup, "ms_per_step": ms_step, "quick": True,
                              "config": config_dict(idx, w, topk, world, ulysses)}))
        if dist is not None:
            if ulysses:
                from spargeattn_b200.sharding import close_peer_exchanges
                close_peer_exchanges()
            dist.destroy_process_group()
        return

    # ---- end-to-end arm: pinned host buffers in, host buffer out, copies inside the timed region
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty_like(hq).pin_memory()
    if ulysses:
        dq, dk, dv = (torch.empty_like(t) for t in (q, k, v))

        def e2e_step():
            dq.copy_(hq, non_blocking=True)
            dk.copy_(hk, non_blocking=True)
            dv.copy_(hv, non_blocking=True)
            ho.copy_(api(dq, dk, dv), non_blocking=True)
    else:
        # the library's host-buffer front end: head chunks pipelined over upload / compute / download streams
        from spargeattn_b200.host import spas_sage2_attn_meansim_topk_host

        def e2e_step():
            spas_sage2_attn_meansim_topk_host(hq, hk, hv, out=ho, device=dev, heads_per_chunk=args.e2e_heads_per_chunk,
                                              topk=topk, is_causal=causal, pvthreshd=args.pvthreshd)

    for _ in range(2):
        e2e_step()
    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e = timed(e2e_step, e2e_steps)
    clk.__exit__()
    e2e_value = total_ops / (ms_e2e * 1e-3) / 1e12
    in_bytes, out_bytes = 3 * q.numel() * 2, q.numel() * 2

    # ---- per-kernel timings on this rank (CUDA events on the launching stream)
    kernels, roofline = {}, None
    if rank == 0 and not ulysses:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        bf16_peak = float(peaks.get("bf16_tflops", 1590.0))
        peak_src = "measured" if peaks else "fallback"
        qc, kc, vc = core._prologue(q, k, v, "HND")
        thr = core.hyperparameter_check(-0.1, H, dev)
        tk = core.hyperparameter_check(topk, H, dev)
        pv = core._pv_threshold_tensor(args.pvthreshd, H, dev)   # None for the API default (test compiled out)
        reps = max(5, min(args.steps, 20))

        def t_kernel(fn):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps

        km = ops.k_mean(kc)
        pq, sq, q8, qs = ops.pool_sim_quant(qc, None, 128, thr)
        pk, sk, k8, ks = ops.pool_sim_quant(kc, km, 64, thr)
        lut, valid, _ = ops.select_blocks(pq, pk, sq, sk, tk, None, causal, False, best_first=pv is None)
        v8, vs = ops.quant_v(vc)
        nd = B * H * N * D
        nq, nk = (N + 127) // 128, (N + 63) // 64
        t = t_kernel(lambda: ops.k_mean(kc))
        kernels["k_mean"] = {"ms": t, "GBps": 2 * nd / t / 1e6, "alg_bytes": 2 * nd}
        t = t_kernel(lambda: ops.pool_sim_quant(qc, None, 128, thr))
        kernels["pool_quant_q"] = {"ms": t, "GBps": 3 * nd / t / 1e6, "alg_bytes": 3 * nd}
        t = t_kernel(lambda: ops.pool_sim_quant(kc, km, 64, thr))
        kernels["pool_quant_k"] = {"ms": t, "GBps": 3 * nd / t / 1e6, "alg_bytes": 3 * nd}
        sel_bytes = B * H * (2 * (nq + nk) * D + nq * nk * 4)
        t = t_kernel(lambda: ops.select_blocks(pq, pk, sq, sk, tk, None, causal, False, best_first=pv is None))
        kernels["select"] = {"ms": t, "GBps": sel_bytes / t / 1e6, "alg_bytes": sel_bytes}
        t = t_kernel(lambda: ops.quant_v(vc))
        kernels["quant_v"] = {"ms": t, "GBps": 3 * nd / t / 1e6, "alg_bytes": 3 * nd}
        out = torch.empty_like(qc)
        attn = lambda: ops.attn_fwd(q8, k8, v8, lut, valid, pv, qs, ks, vs, D ** -0.5, False, qc.dtype, out)
        t_attn = t_kernel(attn)
        live = int(valid.sum().item())
        active_flop = 4.0 * 128 * 64 * D * live
        achieved = active_flop / (t_attn * 1e-3) / 1e12
        peak8 = 2.0 * bf16_peak
        kernels["attn"] = {"ms": t_attn, "active_TOPS": achieved, "live_blocks": live,
                           "density": live / float(B * H * nq * nk)}
        # comparator: the same kernel with every block live = a dense INT8/FP8 attention of this shape
        ones = torch.ones(B, H, nq, nk, dtype=torch.uint8, device=dev)
        lut_d, valid_d = ops.mask_to_lut(ones)
        t_dense = t_kernel(lambda: ops.attn_fwd(q8, k8, v8, lut_d, valid_d, pv, qs, ks, vs, D ** -0.5, False, qc.dtype, out))
        kernels["attn_dense_mask"] = {"ms": t_dense, "dense_TOPS": dense_equiv_ops(B, H, N, D, False) / (t_dense * 1e-3) / 1e12,
                                      "sparse_kernel_speedup": t_dense / t_attn}
        del ones, lut_d, valid_d
        for kname in ("k_mean", "pool_quant_q", "pool_quant_k", "select", "quant_v"):
            kernels[kname]["frac_of_hbm_peak"] = kernels[kname]["GBps"] / hbm_peak
        roofline = {"kernel": "attn_kernel (tcgen05 INT8 QK^T + FP8 PV)", "bound": "tensor", "achieved": achieved,
                    "peak": peak8, "unit": "TFLOP/s", "frac": achieved / peak8,
                    "peak_note": f"2 x {peak_src} dense bf16 burst ({bf16_peak} TFLOP/s); 8-bit nominal is "
                                 f"{NOMINAL_8BIT_TOPS} -> frac_of_nominal {achieved / NOMINAL_8BIT_TOPS:.3f}",
                    "algorithmic_flop_per_launch": active_flop, "launch_ms": t_attn,
                    "traffic": ATTN_DRAM_TRAFFIC_BYTES.get(idx), "hbm_peak_GBps": hbm_peak}
        ops.check_device_status(dev)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tops, full, sample_s, note = cpu_reference_sample(idx, w, topk, q_blocks=1 << 30)
        cpu_baseline = {"value": tops, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": note,
                        "sample_seconds": sample_s}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "strong" if ulysses else "weak",
                "vs_baseline": None, "dtype": "int8-qk/fp8-pv", "data": "synthetic",
                "config": config_dict(idx, w, topk, world, ulysses), "clocks": clk.summary(),
                "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": in_bytes,
                        "d2h_bytes_per_step": out_bytes},
                "gpu_launches": GPU_LAUNCHES_PER_STEP * args.steps * calls_per_step, "roofline": roofline, "kernels": kernels,
                "cpu_baseline": cpu_baseline}
        print(json.dumps(line))
    if dist is not None:
        if ulysses:
            from spargeattn_b200.sharding import close_peer_exchanges
            close_peer_exchanges()
        dist.destroy_process_group()


# kernels of this library launched by one API call: k_mean (2), pool_quant (2), select (1),
# quant_v (3, plus one memset), attention (1)
GPU_LAUNCHES_PER_STEP = 9
# dram bytes (read + write) of one attention launch, from the ncu capture summarised under profiles/
ATTN_DRAM_TRAFFIC_BYTES = {2: 154650112 + 70302464}   # profiles/attn_kernel_cfg2_wan480p.md

if __name__ == "__main__":
    main()
