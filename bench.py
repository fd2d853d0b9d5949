#!/usr/bin/env python
"""Benchmark of the sparse-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload IDX] [--impl ours|reference]

A step is one full call of `spas_sage2_attn_meansim_topk_cuda(q, k, v, topk)` (K mean, predictor, INT8/FP8
quantisers, block-sparse attention) on the synthetic inputs of the named workload; default = workload 2
(Wan2.1-1.3B 480p shape, B=1 H=12 N=32760 D=128 bf16, non-causal, topk 0.5).  Prints ONE JSON line (rank 0).
Metric: dense-equivalent TOPS = 4*B*H*N^2*D / time (causal: half).

With N GPUs the SAME problem is split (strong scaling): the (batch, head, query-block) cells are cut into N
contiguous runs of equal cost (`sharding.partition_rows`), every rank generates and processes only the heads
it touches, no collective on the data path; time = slowest rank, value = whole-problem operations / time.
From 2 GPUs on, the line also carries `ulysses_cfg4`: workload 4 run sequence-parallel (Ulysses all-to-all).

`--impl reference` times the CPU restatement of the reference algorithm (oracle/) on the host cores, one
complete head per step; it never imports this library's package.  The compiled reference itself (its CUDA
kernels built for sm_100, oracle/_ref) is timed on the GPU by a child process and reported under
`reference_on_this_gpu` of the normal line.
"""
import argparse
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))

METRIC = "dense_equivalent_attention_throughput_topk0.5"
# DRAM bytes (read + write) of one attention launch per workload index, as captured by ncu (see profiles/)
ATTN_DRAM_TRAFFIC_FROM_PROFILE = {2: 155120896 + 69793536}
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
    ap.add_argument("--no-extras", action="store_true", help="skip the other workloads, comparators and the reference-on-GPU leg")
    ap.add_argument("--e2e-heads-per-chunk", type=int, default=2)
    ap.add_argument("--quick", action="store_true", help="device-resident arm only (for profiler runs)")
    ap.add_argument("--api", default="sage2", choices=["sage2", "sage1"],
                    help="sage2: spas_sage2_attn_meansim_topk_cuda (INT8 QK, FP8 PV; the benchmark); sage1: the Sage1-signature "
                         "entry point spas_sage_attn_meansim_topk_cuda (fp16 PV, token-level causal), device-resident arm only")
    ap.add_argument("--share", default=None, metavar="R/W",
                    help="single process: run the share that rank R of a W-GPU job would own (the row sharding has no "
                         "collective, so one GPU can time any rank's share); the printed value assumes every rank takes as long")
    return ap.parse_args()


def load_synthetic():
    """spargeattn_b200/synthetic.py by path: the generators need no CUDA library."""
    spec = importlib.util.spec_from_file_location("sparge_synthetic", os.path.join(ROOT, "spargeattn_b200", "synthetic.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def dense_equiv_ops(B, H, N, D, causal):
    ops = 4.0 * B * H * float(N) * float(N) * D
    return ops / 2 if causal else ops


def workload_text(syn, idx, topk, pv):
    w = syn.WORKLOADS[idx]
    B, H, N, D = syn.workload_shape(idx)
    return (f"cfg{idx}:{w['name']} B={B} H={H} N={N} D={D} bf16 {'causal' if w['causal'] else 'non-causal'} "
            f"topk={topk} pvthreshd={pv:g}")


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
def cpu_head_step(O, syn, idx, topk, cache):
    """One complete head of the workload through the CPU restatement: K mean, predictor, quantisers, then
    fp32 attention on the de-quantised operands under the expanded block mask. Returns seconds."""
    w = syn.WORKLOADS[idx]
    _, _, N, D = syn.workload_shape(idx)
    if idx not in cache:
        cache[idx] = syn.workload_heads_qkv(idx, [(0, 0)], "cpu")
    q, k, v = cache[idx]
    t0 = time.perf_counter()
    km = O.k_mean(k)
    pr = O.predictor(q, k, km, w["causal"], -0.1, None, topk, False)
    v8, vs = O.quant_v(v)
    O.attention_dense_masked(pr["q_int8"], pr["q_scale"], pr["k_int8"], pr["k_scale"], v8, vs, pr["map"], D ** -0.5, False,
                             torch.bfloat16, q_chunk=512)
    return time.perf_counter() - t0


def cpu_sample_note(syn, idx):
    B, H, N, D = syn.workload_shape(idx)
    return (f"one complete head per step (1 of {B * H}: heads are independent, the whole call is {B * H} such steps): "
            f"K mean + predictor + INT8/FP8 quantisers + fp32 attention on the de-quantised operands under the expanded "
            f"128x64 block mask; value = that head's dense-equivalent operations / its time")


def run_reference(args):
    """CPU restatement on the host cores, one head per step; nothing of the product is imported."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import sparge_oracle as O
    syn = load_synthetic()
    torch.set_num_threads(os.cpu_count())
    idx = args.workload
    w = syn.WORKLOADS[idx]
    topk = args.topk if args.topk is not None else w["topk"]
    B, H, N, D = syn.workload_shape(idx)
    cache, secs = {}, []
    for i in range(args.warmup + args.steps):
        t = cpu_head_step(O, syn, idx, topk, cache)
        if i >= args.warmup:
            secs.append(t)
    per_step = sum(secs) / len(secs)
    tops = dense_equiv_ops(1, 1, N, D, w["causal"]) / per_step / 1e12
    line = {"impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8-qk/fp8-pv (emulated in fp32 on CPU)", "data": "synthetic",
            "config": {"workload": workload_text(syn, idx, topk, args.pvthreshd), "step": "one head (see cpu_baseline.sample)"},
            "cpu_baseline": {"value": tops, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                             "sample": cpu_sample_note(syn, idx)},
            "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------ GPU arm helpers
def t_gpu(fn, reps, warm=2):
    """CUDA-event time per call on the current stream (the stream every kernel of this library launches on)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def measured_8bit_peaks(ops):
    """tcgen05.mma rates of this GPU (operands resident in shared memory, N = 128 as the attention kernel issues)."""
    i8 = ops.tensor_peak("i8", 128, 2, 40.0)
    f8 = ops.tensor_peak("f8", 128, 2, 40.0)
    combined = 2.0 / (1.0 / i8["tops"] + 1.0 / f8["tops"])      # half of the kernel's operations are INT8, half FP8
    return i8["tops"], f8["tops"], combined


def attention_parts(S, core, ops, q, k, v, topk, causal, pvthreshd, reps):
    """Per-kernel times of one call and the attention kernel's active-block rate."""
    B, H, N, D = q.shape
    dev = q.device
    qc, kc, vc = core._prologue(q, k, v, "HND")
    thr = core.hyperparameter_check(-0.1, H, dev)
    tk = core.hyperparameter_check(topk, H, dev)
    pv = core._pv_threshold_tensor(pvthreshd, H, dev)       # None for the API default (test compiled out)
    km = ops.k_mean(kc)
    pq, sq, q8, qs = ops.pool_sim_quant(qc, None, 128, thr)
    pk, sk, k8, ks = ops.pool_sim_quant(kc, km, 64, thr)
    lut, valid, _ = ops.select_blocks(pq, pk, sq, sk, tk, None, causal, False, best_first=pv is None)
    v8, vs = ops.quant_v(vc)
    nd = B * H * N * D
    nq, nk = (N + 127) // 128, (N + 63) // 64
    kern = {}
    t = t_gpu(lambda: ops.k_mean(kc), reps)
    kern["k_mean"] = {"ms": t, "GBps": 2 * nd / t / 1e6, "alg_bytes": 2 * nd}
    t = t_gpu(lambda: ops.pool_sim_quant(qc, None, 128, thr), reps)
    kern["pool_quant_q"] = {"ms": t, "GBps": 3 * nd / t / 1e6, "alg_bytes": 3 * nd}
    t = t_gpu(lambda: ops.pool_sim_quant(kc, km, 64, thr), reps)
    kern["pool_quant_k"] = {"ms": t, "GBps": 3 * nd / t / 1e6, "alg_bytes": 3 * nd}
    sel_bytes = B * H * (2 * (nq + nk) * D + nq * nk * 4)
    t = t_gpu(lambda: ops.select_blocks(pq, pk, sq, sk, tk, None, causal, False, best_first=pv is None), reps)
    kern["select"] = {"ms": t, "GBps": sel_bytes / t / 1e6, "alg_bytes": sel_bytes}
    t = t_gpu(lambda: ops.quant_v(vc), reps)
    kern["quant_v"] = {"ms": t, "GBps": 3 * nd / t / 1e6, "alg_bytes": 3 * nd}
    out = torch.empty_like(qc)
    t_attn = t_gpu(lambda: ops.attn_fwd(q8, k8, v8, lut, valid, pv, qs, ks, vs, D ** -0.5, False, qc.dtype, out), reps)
    live = int(valid.sum().item())
    active_flop = 4.0 * 128 * 64 * D * live
    kern["attn"] = {"ms": t_attn, "active_TOPS": active_flop / (t_attn * 1e-3) / 1e12, "live_blocks": live,
                    "density": live / float(B * H * nq * nk), "active_flop": active_flop,
                    # operand bytes one launch has to move at least once: INT8 Q and K, FP8 V, the LUT rows and the output
                    "alg_bytes": 2 * nd + B * H * nq * 128 * D + 4 * live + 2 * nd}
    parts = dict(q8=q8, k8=k8, v8=v8, qs=qs, ks=ks, vs=vs, pv=pv, qc=qc, out=out)
    return kern, parts


def config_row(S, core, ops, syn, idx, topk, pvthreshd, dev, peak8, reps=5):
    """One workload through the public API on this GPU: call latency, dense-equivalent and active-block rates."""
    w = syn.WORKLOADS[idx]
    B, H, N, D = syn.workload_shape(idx)
    heads = [(b, h) for b in range(B) for h in range(H)]
    q, k, v = (t.view(B, H, N, D) for t in syn.workload_heads_qkv(idx, heads, dev))
    api = lambda: S.spas_sage2_attn_meansim_topk_cuda(q, k, v, topk=topk, is_causal=w["causal"], pvthreshd=pvthreshd)
    ms = t_gpu(api, reps, warm=3)
    kern, _ = attention_parts(S, core, ops, q, k, v, topk, w["causal"], pvthreshd, reps)
    a = kern["attn"]
    row = {"workload": workload_text(syn, idx, topk, pvthreshd), "api_ms": ms,
           "dense_equiv_TOPS": dense_equiv_ops(B, H, N, D, w["causal"]) / ms / 1e9, "attn_ms": a["ms"],
           "active_TOPS": a["active_TOPS"], "frac_of_measured_8bit_peak": a["active_TOPS"] / peak8,
           "density": a["density"],
           "preprocess_ms": sum(kern[n]["ms"] for n in ("k_mean", "pool_quant_q", "pool_quant_k", "select", "quant_v"))}
    if idx == 1:    # the same shape through block_sparse_sage2_attn_cuda with a Bernoulli(0.4) block mask, diagonal forced
        mask = syn.bernoulli_block_mask(B, H, N, 0.4, 1, dev)
        t = t_gpu(lambda: S.block_sparse_sage2_attn_cuda(q, k, v, mask_id=mask), reps, warm=3)
        row["block_sparse_api_ms"] = t
        row["block_sparse_dense_equiv_TOPS"] = dense_equiv_ops(B, H, N, D, False) / t / 1e9
        row["block_sparse_density"] = float(mask.float().mean().item())
    del q, k, v
    torch.cuda.empty_cache()
    return row


def reference_on_gpu(workloads):
    """The compiled reference timed by a child process (its modules never share a process with this library)."""
    script = os.path.join(ROOT, "oracle", "time_reference.py")
    if not os.path.isdir(os.path.join(ROOT, "oracle", "_ref", "spas_sage_attn")):
        return {"unavailable": "oracle/_ref is not present (built by oracle/build_ref.py where the reference checkout is)"}
    try:
        r = subprocess.run([sys.executable, script, "--workloads", ",".join(str(i) for i in workloads), "--block-sparse",
                            "--steps", "5"], capture_output=True, text=True, timeout=600)
        rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
        if not rows:
            err = r.stderr.strip().splitlines()
            return {"unavailable": "reference run produced no result: " + (err[-1][:200] if err else "no output")}
        return {"rows": rows, "how": "child process `python oracle/time_reference.py`, CUDA events, 5 steps after 3 warm-ups"}
    except Exception as e:   # a broken reference leg must not take the benchmark line with it
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


def _cpu_list(text):
    cpus = []
    for part in text.strip().split(","):
        a, _, b = part.partition("-")
        cpus += list(range(int(a), int(b or a) + 1))
    return cpus


def bind_to_gpu_numa_node(local):
    """Pin this process (and the pinned host buffers it allocates afterwards: pages are placed on first touch) to the
    CPU cores next to the GPU. The cores come from sysfs (the PCI device's NUMA node) or, where a container hides
    that, from the CPU-affinity column of `nvidia-smi topo -m`. Returns what was done, or None."""
    allowed = os.sched_getaffinity(0)

    def bind(cpus, how):
        cpus = set(cpus) & allowed
        if not cpus or cpus == allowed:
            return None
        os.sched_setaffinity(0, cpus)
        return f"{len(cpus)} cpus ({how})"

    try:
        p = torch.cuda.get_device_properties(local)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
        if node >= 0:
            done = bind(_cpu_list(open(f"/sys/devices/system/node/node{node}/cpulist").read()), f"sysfs numa node {node}")
            if done:
                return done
    except Exception:
        pass
    try:
        out = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20).stdout
        rows = [[c.strip() for c in line.split("\t")] for line in out.splitlines() if line.strip()]
        header = next(r for r in rows if "CPU Affinity" in r)
        col = header.index("CPU Affinity")
        # data rows carry the row label in front, so their columns are shifted by one against a header that starts
        # with an empty cell; take the cell that parses as a cpu list at or next to the header's position
        row = next(r for r in rows if r and r[0] == f"GPU{local}")
        for c in (col, col + 1, col - 1):
            if 0 <= c < len(row) and row[c] and all(ch.isdigit() or ch in ",-" for ch in row[c]):
                return bind(_cpu_list(row[c]), "nvidia-smi topo")
    except Exception:
        pass
    return None


# ------------------------------------------------------------------------------------------ GPU arm
def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    # in-switch (NVLS) reductions are not needed by anything here, and a rank that dies while bound to an NVLink
    # multicast object disturbs its peers' GPUs: keep NCCL on plain peer transfers
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

    import spargeattn_b200 as S
    from spargeattn_b200 import core, ops, sharding, synthetic as syn
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = bind_to_gpu_numa_node(local) if world > 1 else None
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    idx = args.workload
    w = syn.WORKLOADS[idx]
    topk = args.topk if args.topk is not None else w["topk"]
    causal = w["causal"]
    B, H, N, D = syn.workload_shape(idx)
    nq = (N + 127) // 128

    # ---- this rank's share: contiguous runs of (batch, head, query block) cells of equal expected cost
    n_sel = max(1, int(topk * ((N + 63) // 64)))
    row_cost = [min(n_sel, 2 * (i + 1)) for i in range(nq)] if causal else None
    part_rank, part_world = rank, world
    if args.share:
        assert world == 1, "--share is for a single process"
        part_rank, part_world = (int(x) for x in args.share.split("/"))
        assert 0 <= part_rank < part_world
    units = sharding.partition_rows(B, H, nq, part_world, row_cost)[part_rank]
    heads = [(b, h) for (b, h, _, _) in units]
    q, k, v = syn.workload_heads_qkv(idx, heads, dev)                  # [1, Hloc, N, D]
    whole = all(a == 0 and n == nq for (_, _, a, n) in units)
    ranges = torch.tensor([[a, n] for (_, _, a, n) in units], dtype=torch.int32).view(1, len(units), 2)
    ranges_dev, ranges_max = ranges.to(dev), int(ranges[..., 1].max())
    if args.api == "sage1":
        assert whole and args.quick, "--api sage1 times whole heads, device-resident arm only (--quick)"
        api = lambda a, b, c: S.spas_sage_attn_meansim_topk_cuda(a, b, c, topk=topk, is_causal=causal,
                                                                pvthreshd=args.pvthreshd)
    elif whole:     # every owned head is complete: the public entry point itself
        api = lambda a, b, c: S.spas_sage2_attn_meansim_topk_cuda(a, b, c, topk=topk, is_causal=causal,
                                                                 pvthreshd=args.pvthreshd)
    else:
        api = lambda a, b, c: sharding.attention_units(a, b, c, ranges_dev, ranges_max, topk=topk, is_causal=causal,
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
    for _ in range(max(args.warmup, 3)):
        api(q, k, v)
    clk = ClockSampler(local)
    clk.__enter__()
    ms_step = timed(lambda: api(q, k, v), args.steps)
    ops.check_device_status(dev)
    total_ops = dense_equiv_ops(B, H, N, D, causal)
    value = total_ops / (ms_step * 1e-3) / 1e12
    config = {"workload": workload_text(syn, idx, topk, args.pvthreshd),
              "sharding": (f"strong scaling over {part_world} GPU(s): (batch, head, query-block) cells cut into {part_world} contiguous "
                           f"runs of equal cost, no collective; rank {part_rank} owns {[list(u) for u in units]} as (b, h, first block, blocks)"),
              "l2_policy": "inputs larger than L2 on every rank (q,k,v = %.0f MB on rank 0; L2 126 MB)" % (3 * q.numel() * 2 / 1e6)}

    if args.quick:
        clk.__exit__()
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                              "warmup": args.warmup, "ms_per_step": ms_step, "quick": True, "config": config}))
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- end-to-end arm: pinned host buffers in, host buffer out, copies inside the timed region
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty_like(hq).pin_memory()
    # the library's host-buffer front end: head chunks pipelined over upload / compute / download streams; a rank
    # that owns part of a head moves only its query rows and its rows of the result
    from spargeattn_b200.host import spas_sage2_attn_meansim_topk_host

    def e2e_step():
        spas_sage2_attn_meansim_topk_host(hq, hk, hv, out=ho, device=dev, units=None if whole else units,
                                          heads_per_chunk=args.e2e_heads_per_chunk if whole else 1,
                                          topk=topk, is_causal=causal, pvthreshd=args.pvthreshd)

    for _ in range(3):
        e2e_step()
    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e = timed(e2e_step, e2e_steps)
    clk.__exit__()
    e2e_value = total_ops / (ms_e2e * 1e-3) / 1e12
    own_rows = sum(min((a + n) * 128, N) - a * 128 for (_, _, a, n) in units)      # query rows this rank owns
    in_bytes, out_bytes = (own_rows + 2 * len(units) * N) * D * 2, own_rows * D * 2    # owned q rows + whole k, v / owned o rows
    if dist is not None:       # bytes of the whole job per step
        t = torch.tensor([float(in_bytes), float(out_bytes)], device=dev)
        dist.all_reduce(t)
        in_bytes, out_bytes = int(t[0].item()), int(t[1].item())

    # ---- per-kernel timings and the roofline of the dominant kernel (rank 0, its own share of the problem)
    kernels, roofline, extras = {}, None, {}
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        bf16_peak = float(peaks.get("bf16_tflops", 1590.0))
        peak_src = "measured" if peaks else "fallback"
        reps = max(5, min(args.steps, 20))
        kernels, parts = attention_parts(S, core, ops, q, k, v, topk, causal, args.pvthreshd, reps)
        # the peak probe loads the tensor pipe for ~0.1 s and can pull the clocks down for a moment: it runs after
        # the kernels have been timed, and the other workloads below start with their own warm-up calls
        i8_peak, f8_peak, peak8 = measured_8bit_peaks(ops)
        for kname in ("k_mean", "pool_quant_q", "pool_quant_k", "select", "quant_v"):
            kernels[kname]["frac_of_hbm_peak"] = kernels[kname]["GBps"] / hbm_peak
        a = kernels["attn"]
        roofline = {"kernel": "attn_kernel (tcgen05 INT8 QK^T + FP8 PV)", "bound": "tensor", "achieved": a["active_TOPS"],
                    "peak": peak8, "unit": "TFLOP/s", "frac": a["active_TOPS"] / peak8,
                    "peak_note": (f"measured in this run with sparge_tensor_peak (tcgen05.mma M=128 N=128 K=32 from shared "
                                  f"memory, two issuing CTAs per SM, ~40 ms each): kind::i8 {i8_peak:.0f}, kind::f8f6f4 "
                                  f"{f8_peak:.0f} TOPS; the kernel does half of its operations in each, so peak = their "
                                  f"harmonic mean. For context: 2 x {peak_src} dense bf16 burst = {2 * bf16_peak:.0f}, "
                                  f"vendor nominal {NOMINAL_8BIT_TOPS:.0f} (frac_of_nominal {a['active_TOPS'] / NOMINAL_8BIT_TOPS:.3f})"),
                    "algorithmic_flop_per_launch": a["active_flop"], "launch_ms": a["ms"],
                    "traffic": ATTN_DRAM_TRAFFIC_FROM_PROFILE.get(idx) if world == 1 else None,
                    "traffic_note": ("dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload, from the ncu "
                                     "capture summarised in profiles/attn_kernel_cfg2_wan480p.md (a recorded figure, not measured "
                                     f"by this run); algorithmic operand bytes of this launch: {a['alg_bytes']}"),
                    "hbm_peak_GBps": hbm_peak}
        if world == 1 and not args.no_extras:
            nk = (N + 63) // 64
            # comparator 1: the same kernel with every block live = a dense INT8/FP8 attention of this shape
            ones = torch.ones(1, q.shape[1], nq, nk, dtype=torch.uint8, device=dev)
            lut_d, valid_d = ops.mask_to_lut(ones)
            t_dense = t_gpu(lambda: ops.attn_fwd(parts["q8"], parts["k8"], parts["v8"], lut_d, valid_d, parts["pv"], parts["qs"],
                                                 parts["ks"], parts["vs"], D ** -0.5, False, parts["qc"].dtype, parts["out"]), reps)
            del ones, lut_d, valid_d
            # comparator 2 (independent): torch's bf16 scaled_dot_product_attention on the same q, k, v
            t_sdpa = t_gpu(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal), reps)
            extras["dense_comparators"] = {
                "own_kernel_all_blocks_live": {"ms": t_dense, "dense_TOPS": total_ops / (t_dense * 1e-3) / 1e12},
                "torch_sdpa_bf16": {"ms": t_sdpa, "dense_TOPS": total_ops / (t_sdpa * 1e-3) / 1e12},
                "api_call_vs_own_dense_kernel": t_dense / ms_step, "api_call_vs_torch_sdpa": t_sdpa / ms_step,
                "attn_kernel_vs_own_dense_kernel": t_dense / a["ms"]}
            del parts
            torch.cuda.empty_cache()
            rows = {}
            if idx == 2:
                for tk_, pv_ in ((0.3, 50.0), (0.7, 50.0), (0.5, 5.0)):
                    rows[f"cfg2_topk{tk_:g}_pv{pv_:g}"] = config_row(S, core, ops, syn, 2, tk_, pv_, dev, peak8)
            del q, k, v
            torch.cuda.empty_cache()
            for j in (0, 1, 3, 4):
                if j != idx:
                    rows[f"cfg{j}"] = config_row(S, core, ops, syn, j, syn.WORKLOADS[j]["topk"], 50.0, dev, peak8)
            extras["configs"] = rows
            extras["reference_on_this_gpu"] = reference_on_gpu([0, 1, 2, 3, 4])
        ops.check_device_status(dev)

    # ---- workload 4 sequence-parallel (Ulysses) as an extra measurement from 2 GPUs on
    if world > 1 and not args.no_extras:
        extras["ulysses_cfg4"] = run_ulysses_cfg4(S, syn, sharding, ops, dist, dev, rank, world)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import sparge_oracle as O
        torch.set_num_threads(os.cpu_count())
        cache = {}
        cpu_head_step(O, syn, idx, topk, cache)                      # warm-up (allocator, thread pool)
        secs = [cpu_head_step(O, syn, idx, topk, cache) for _ in range(3)]
        per = sum(secs) / len(secs)
        cpu_baseline = {"value": dense_equiv_ops(1, 1, N, D, causal) / per / 1e12, "unit": UNIT, "cores": os.cpu_count(),
                        "kind": "port", "sample": cpu_sample_note(syn, idx) + f"; 3 timed heads, {per:.2f} s each",
                        "sample_seconds": sum(secs)}

    if rank == 0:
        # kernels of this library launched by one API call: k_mean (2), pool_quant (2), select (1),
        # quant_v (3), attention (1); counted per timed step of the device-resident arm
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "int8-qk/fp8-pv", "data": "synthetic", "config": config,
                "clocks": clk.summary(),
                "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": in_bytes,
                        "d2h_bytes_per_step": out_bytes, "numa_node_bound": numa},
                "gpu_launches": 9 * args.steps * world, "roofline": roofline, "kernels": kernels,
                "cpu_baseline": cpu_baseline}
        if args.share:
            line["share_of"] = args.share
        line.update(extras)
        print(json.dumps(line))
    if dist is not None:
        sharding.close_peer_exchanges()
        dist.destroy_process_group()


def run_ulysses_cfg4(S, syn, sharding, ops, dist, dev, rank, world):
    """Workload 4 (B=1 H=24 N=119056 D=128, topk 0.4) sequence-parallel: every rank holds N/G tokens of all heads."""
    try:
        idx = 4
        w = syn.WORKLOADS[idx]
        B, H, N, D = syn.workload_shape(idx)
        if N % world or H % world:
            return {"skipped": f"N={N} or H={H} not divisible by {world}"}
        n_loc = N // world
        heads = [(0, h) for h in range(H)]
        # every rank generates the same per-head tensors and keeps its own token slice (one head at a time: 90 MB)
        qs, ks, vs = [], [], []
        for hd in heads:
            a, b, c = syn.workload_heads_qkv(idx, [hd], dev)
            qs.append(a[:, :, rank * n_loc:(rank + 1) * n_loc].clone())
            ks.append(b[:, :, rank * n_loc:(rank + 1) * n_loc].clone())
            vs.append(c[:, :, rank * n_loc:(rank + 1) * n_loc].clone())
            del a, b, c
        q, k, v = (torch.cat(t, 1) for t in (qs, ks, vs))
        del qs, ks, vs
        fn = lambda: sharding.ulysses_attention(q, k, v, topk=w["topk"], is_causal=False)
        for _ in range(3):
            o = fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        steps = 5
        e0.record()
        for _ in range(steps):
            o = fn()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        # byte equality of head 0 with a single-GPU call: rank 0 gathers head 0's output slices and recomputes it alone
        parts = [torch.empty_like(o[:, :1]) for _ in range(world)]
        dist.all_gather(parts, o[:, :1].contiguous())
        equal = None
        if rank == 0:
            a, b, c = syn.workload_heads_qkv(idx, [(0, 0)], dev)
            ref = S.spas_sage2_attn_meansim_topk_cuda(a, b, c, topk=w["topk"])
            equal = bool(torch.equal(torch.cat(parts, 2), ref))
        ops.check_device_status(dev)
        return {"ms_per_step": ms, "dense_equiv_TOPS": dense_equiv_ops(B, H, N, D, False) / ms / 1e9, "n_gpus": world,
                "tokens_per_rank": n_loc, "heads_per_rank_inside": H // world, "steps": steps,
                "head0_bytes_equal_to_single_gpu_call": equal}
    except Exception as e:
        return {"failed": f"{type(e).__name__}: {e}"[:300]}


if __name__ == "__main__":
    main()
