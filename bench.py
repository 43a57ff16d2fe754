#!/usr/bin/env python3
"""Benchmark of the NSA layer hot path (forward + backward) on B200.

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --gpus N ...            # the reference algorithm on the host CPU

Workload (BASELINE.json's metric): one NSA layer forward + backward at T = 65536, H = 64 query heads,
G = 4 KV groups, dk = 192, dv = 128, window 512, l = 32, d = 16, l' = 64, n = 16 (3 forced blocks),
sigmoid gates, d_model = 2560, bf16, synthetic seeded inputs (keys carry a per-64-token-block offset).
One sequence per GPU (weak scaling); with N > 1 the only collective is the NCCL all-reduce of the
compression-MLP and gate-MLP weight gradients, inside the timed step.

Prints ONE JSON line (rank 0).  `value` = tokens/s with inputs resident in HBM; `e2e` = the same step
fed from pinned host buffers each step (host->device copies and a device->host read of the result
inside the timed region); `roofline` = the dominant kernel against the measured bf16 tensor peak;
`cpu_baseline` = the CPU oracle (a restatement of the reference's algorithm) on a bounded sample.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "nsa-test_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

CFG = dict(H=64, G=4, dk=192, dv=128, w=512, l=32, d=16, l_prime=64, n=16, d_model=2560)
METRIC = "NSA layer fwd+bwd tokens/s at T=64K"


# dram__bytes_read.sum + dram__bytes_write.sum per launch from an ncu capture at T=8192, per (group, query, slot) unit of
# the selection kernels.  That case is too small to be captured at full size under the
# capture-size rule, so the figure is scaled by the units of the workload; at T=8192 62 % of the gathers hit L2, at
# T=65536 fewer do, so the scaled figure is a lower bound of the full-size traffic.
NCU_DRAM_BYTES_PER_UNIT = {"slc_bwd_fused": (3497088000 + 3072542000) / (8192 * 4 * 16),
                           "slc_fwd": (1598514000 + 2035920000) / (8192 * 4 * 16)}


def selection_bytes_per_unit(kernel):
    """Algorithmic HBM bytes of one (group, query, slot) unit of the selection kernels: every unit gathers the query's
    rows of all heads of the group (forward: Q; backward: Q and dO) and writes one partial (forward: normalised O rows and
    two statistics per head; backward: dQ rows); the key/value blocks and the inverse index are 1 % of that."""
    c = CFG
    hpg = c["H"] // c["G"]
    if kernel == "slc_fwd":
        return hpg * (c["dk"] * 2 + c["dv"] * 2 + 8)
    return hpg * ((c["dk"] + c["dv"]) * 2 + c["dk"] * 2)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(tflops=d.get("bf16_tflops", 1590.0), tflops_sustained=d.get("bf16_tflops_sustained", 1400.0),
                    hbm_gbs=d.get("hbm_gbs", 6650.0), source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """nvidia-smi SM clock / throttle-reason samples while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for nme, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nme)
        sm.sort()
        busy = sm[len(sm) // 2:] if sm else []          # upper half = samples taken under load
        med = busy[len(busy) // 2] if busy else None
        return dict(sm_mhz=med, sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm))


# --------------------------------------------------------------------------------------------------
# workload
# --------------------------------------------------------------------------------------------------

def make_device_inputs(T, dev, seed, B=1):
    c = CFG
    g = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *s, std=1.0: torch.randn(*s, generator=g, device=dev) * std
    q = rn(B, c["H"], T, c["dk"]).bfloat16()
    k = rn(B, c["G"], c["dk"], T)
    off = rn(B, c["G"], c["dk"], T // c["l_prime"], std=0.5)
    k = (k + off.repeat_interleave(c["l_prime"], dim=-1)).bfloat16()
    v = rn(B, c["G"], T, c["dv"]).bfloat16()
    do = rn(B, c["H"], T, c["dv"]).bfloat16()
    x = rn(B, T, c["d_model"]).bfloat16()
    dk, l = c["dk"], c["l"]
    params = dict(pos_embed=rn(l, l, std=0.02), w1=rn(2 * dk, dk + l, std=0.02), b1=torch.zeros(2 * dk, device=dev),
                  w2=rn(dk, 2 * dk, std=0.02), b2=torch.zeros(dk, device=dev),
                  gw1=rn(c["d_model"] // 2, c["d_model"], std=0.02).bfloat16(), gb1=torch.zeros(c["d_model"] // 2, device=dev).bfloat16(),
                  gw2=rn(3 * c["H"], c["d_model"] // 2, std=0.02).bfloat16(), gb2=torch.zeros(3 * c["H"], device=dev).bfloat16())
    for p_ in params.values():
        p_.requires_grad_(True)
    return dict(q=q, k=k, v=v, do=do, x=x), params


def layer_step(inp, params, cfg, world, before_backward=None):
    """One forward + backward of the layer; returns a scalar tensor summarising the result."""
    from nsa.kernels import _GateMLP, nsa_layer
    q = inp["q"].detach().requires_grad_(True)
    k = inp["k"].detach().requires_grad_(True)
    v = inp["v"].detach().requires_grad_(True)
    logits = _GateMLP.apply(inp["x"], params["gw1"], params["gb1"], params["gw2"], params["gb2"])    # gate MLP through the library
    phi = (params["pos_embed"], params["w1"], params["b1"], params["w2"], params["b2"])
    out = nsa_layer(q, k, v, logits, phi, cfg)
    plist = list(params.values())
    if before_backward is not None:
        before_backward()           # the upstream gradient is first needed here
    grads = torch.autograd.grad(out, [q, k, v] + plist, inp["do"])
    if world > 1:
        from nsa.sharding import allreduce_grads
        allreduce_grads(grads[3:])      # phi and gate-MLP weight gradients: the only collective of the layer
    return out[0, 0, -1, :8].float().sum() + grads[0][0, 0, -1, :8].float().sum()


def layer_step_query_sharded(inp, params, cfg, world, before_backward=None):
    """Long-context mode: `inp` holds this rank's slice of the positions; K/V are all-gathered inside the layer and
    their gradients come back reduce-scattered (nsa.sharding.query_sharded_layer)."""
    from nsa.kernels import _GateMLP
    from nsa.sharding import allreduce_grads, query_sharded_layer
    bounds = inp.get("bounds")
    q = inp["q"].detach().requires_grad_(True)
    k = inp["k"].detach().requires_grad_(True)
    v = inp["v"].detach().requires_grad_(True)
    logits = _GateMLP.apply(inp["x"], params["gw1"], params["gb1"], params["gw2"], params["gb2"])
    phi = (params["pos_embed"], params["w1"], params["b1"], params["w2"], params["b2"])
    out = query_sharded_layer(q, k, v, logits, phi, cfg, bounds=bounds)
    plist = list(params.values())
    if before_backward is not None:
        before_backward()           # the upstream gradient is first needed here
    grads = torch.autograd.grad(out, [q, k, v] + plist, inp["do"])
    if world > 1:
        allreduce_grads(grads[3:])
    return out[0, 0, -1, :8].float().sum() + grads[0][0, 0, -1, :8].float().sum()


# Cost of a query that does not depend on its position (sliding window, selected blocks, gate/mix, its share of phi), in
# units of one visible compressed key, for the work-balanced position split.  Fitted to the kernel time each of two ranks
# spent on its slice of a T=65536 sequence (39808 rows: 41.7 ms, the other 25728: 38.2 ms): 0.78 us per query plus
# 13.4 ps per (query, earlier position), i.e. 0.78 us / (13.4 ps * d) at d = 16.
POSITION_INDEPENDENT_COST = 3650.0


def long_context_leg(args, cfg, dev, world, rank, T, headline_ms):
    """Long-context mode inside a multi-GPU run: ONE sequence of T tokens split by position over the ranks (K/V and
    the compressed K/V all-gathered, their gradients reduce-scattered), 5 warm-up + 10 timed steps, device-timed, max
    over ranks.  `headline_ms`: this run's time for one whole T=65536 sequence on one GPU (the weak-scaling step), the
    one-GPU reference of the speed-up at that length."""
    import torch.distributed as dist
    from nsa import sharding
    c = CFG
    inp, params = make_device_inputs(T, dev, seed=0)            # the same sequence on every rank; each keeps its slice
    one_gpu_ms = headline_ms if T == args.T else None
    if one_gpu_ms is None:
        # no one-GPU step of this length has been timed in this run: every rank times the whole sequence on its own GPU
        # (world=1: no collective), 1 warm-up + 2 timed steps, max over ranks
        layer_step(inp, params, cfg, 1)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(2):
            layer_step(inp, params, cfg, 1)
        b.record()
        torch.cuda.synchronize()
        t1 = torch.tensor([a.elapsed_time(b) / 2], device=dev)
        dist.all_reduce(t1, op=dist.ReduceOp.MAX)
        one_gpu_ms = t1.item()
        torch.cuda.empty_cache()
    bounds = sharding.balanced_query_bounds(T, world, POSITION_INDEPENDENT_COST, c["d"])
    t0, t1 = bounds[rank], bounds[rank + 1]
    inp = dict(q=inp["q"][:, :, t0:t1].contiguous(), k=inp["k"][..., t0:t1].contiguous(), v=inp["v"][:, :, t0:t1].contiguous(),
               do=inp["do"][:, :, t0:t1].contiguous(), x=inp["x"][:, t0:t1].contiguous(), bounds=bounds)
    torch.cuda.empty_cache()
    for _ in range(5):
        layer_step_query_sharded(inp, params, cfg, world)
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps = 10
    e0.record()
    for _ in range(steps):
        layer_step_query_sharded(inp, params, cfg, world)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    mine = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    t_ms = mine.clone()
    dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    # every rank's own kernel time for its slice (events around each launch of the library, collectives and waits
    # for other ranks excluded): how even the position split is
    from nsa import _lib
    own = torch.zeros(world, device=dev)
    prof = _lib.profile_kernels(lambda: layer_step_query_sharded(inp, params, cfg, world))
    own[rank] = sum(ms_ for _, ms_ in prof.values())
    dist.all_reduce(own)
    # the exchange steps alone (same tensors, same collectives as inside the layer), device-timed, max over ranks
    sizes = [bounds[i + 1] - bounds[i] for i in range(world)]
    kk, vv = inp["k"].detach().requires_grad_(True), inp["v"].detach().requires_grad_(True)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    for rep in range(3):
        kk.grad = vv.grad = None
        ev[0].record()
        kf, vf = sharding.all_gather_seq(kk, -1, None, sizes), sharding.all_gather_seq(vv, 2, None, sizes)
        ev[1].record()
        torch.autograd.backward([kf, vf], [torch.ones_like(kf), torch.ones_like(vf)])
        ev[2].record()
    torch.cuda.synchronize()
    coll = torch.tensor([ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])], device=dev)
    dist.all_reduce(coll, op=dist.ReduceOp.MAX)
    ms = t_ms.item()
    kv_bytes = c["G"] * T * (c["dk"] + c["dv"]) * 2
    return dict(T=T, n_gpus=world, steps=steps, warmup=5, ms_per_step=round(ms, 3), tokens_per_s=round(T / (ms * 1e-3), 1),
                speedup_vs_n1=round(one_gpu_ms / ms, 3), n1_ms_per_step=round(one_gpu_ms, 3),
                n1_reference="this run's one-GPU step for a whole sequence of the same length" + (
                    "" if T == args.T else " (every rank alone on its GPU, 2 steps after 1 warm-up, max over ranks)"),
                allgather_ms=round(coll[0].item(), 3), reduce_scatter_ms=round(coll[1].item(), 3),
                allgather_bytes=kv_bytes, reduce_scatter_bytes=2 * kv_bytes,
                slices=[bounds[i + 1] - bounds[i] for i in range(world)], rank_kernel_ms=[round(x, 2) for x in own.tolist()])


def attention_flops(T):
    """Algorithmic attention FLOPs per sequence (masked-out keys do not count): forward 2(dk+dv)N,
    backward 2(3dk+2dv)N per (head, query) with N valid keys; selection counted at n full blocks minus
    the causal clipping of the block holding the query."""
    c = CFG
    H, dk, dv, w, l, d, lp, n = c["H"], c["dk"], c["dv"], c["w"], c["l"], c["d"], c["l_prime"], c["n"]
    t = torch.arange(T, dtype=torch.float64)
    n_win = torch.clamp(t + 1, max=w).sum().item()
    n_cmp = torch.clamp(torch.floor((t - l + 1) / d) + 1, min=0).sum().item()
    blocks_visible = torch.floor(t / lp) + 1
    full = torch.clamp(blocks_visible - 1, max=n - 1)                 # earlier blocks, fully visible
    n_slc = (full * lp + (t % lp) + 1).sum().item()
    per_key = dict(fwd=2 * (dk + dv), bwd=2 * (3 * dk + 2 * dv))
    return {br: {ph: per_key[ph] * cnt * H for ph in per_key} for br, cnt in (("win", n_win), ("cmp", n_cmp), ("slc", n_slc))}


def kernel_flops(T):
    """Algorithmic FLOPs of one launch of each tensor-core kernel family (what that kernel's role requires)."""
    c = CFG
    dk, dv = c["dk"], c["dv"]
    a = attention_flops(T)
    unit = {br: a[br]["fwd"] / (2 * (dk + dv)) for br in a}            # (head, query, key) triples
    f = {}
    for br in ("win", "cmp"):
        f[f"fa_fwd_{br}"] = unit[br] * 2 * (dk + dv)
        f[f"fa_bwd_dq_{br}"] = unit[br] * 2 * (2 * dk + dv)             # S, dP, dQ
        f[f"fa_bwd_dkv_{br}"] = unit[br] * 2 * (2 * dk + 2 * dv)        # S^T, dP^T, dV, dK
        f[f"fa_bwd_dqds_{br}"] = unit[br] * 2 * dk                      # dQ from the dS^T tiles the dK/dV kernel left
    f["fa_fwd_cmp_exact"] = f["fa_fwd_cmp"]                            # keys as hi + lo halves: same role, 1.6x the MMAs
    f["slc_fwd"] = unit["slc"] * 2 * (dk + dv)
    f["slc_bwd_fused"] = unit["slc"] * 2 * (3 * dk + 2 * dv)           # S, dP, dQ, dV, dK
    return f


# --------------------------------------------------------------------------------------------------
# CPU arm: the oracle (port of the reference's algorithm) on a bounded sample of the workload
# --------------------------------------------------------------------------------------------------

def cpu_oracle_tokens_per_s(T_sample, steps, threads):
    from oracle import nsa_oracle as O
    c = CFG
    torch.set_num_threads(threads)
    inp = O.make_inputs(1, c["H"], c["G"], T_sample, c["dk"], c["dv"], c["d_model"], c["l"], seed=0, block_offset_std=0.5,
                        l_prime=c["l_prime"], dtype=torch.bfloat16)
    times = []
    for _ in range(steps):
        q, k, v = (inp[n_].clone().requires_grad_(True) for n_ in ("q", "k", "v"))
        t0 = time.perf_counter()
        r = O.nsa_layer(q, k, v, inp["x"], inp["phi"], inp["gate"], l=c["l"], d=c["d"], l_prime=c["l_prime"], n=c["n"], w=c["w"])
        torch.autograd.grad(r["out"], (q, k, v), inp["do"])
        times.append(time.perf_counter() - t0)
    return T_sample / (sum(times) / len(times)), sum(times) / len(times)


def sampled_parity(inp, params, cfg, rows=192):
    """The timed workload itself against the oracle: one extra forward of the CUDA layer, then the CPU oracle (checker
    only) on `rows` sampled query positions, the boundary rows of every branch included.  Block ids must agree outside
    the ambiguity set (rows whose ranking hinges on fp32 rounding order); the branch outputs are compared on every
    sampled row, the oracle attending the blocks the CUDA path chose."""
    from nsa.kernels import nsa_layer
    from oracle import nsa_oracle as O
    c = CFG
    lin = torch.nn.functional.linear
    with torch.no_grad():
        logits = lin(torch.relu(lin(inp["x"], params["gw1"], params["gb1"])), params["gw2"], params["gb2"])
        phi_dev = (params["pos_embed"], params["w1"], params["b1"], params["w2"], params["b2"])
        _, info = nsa_layer(inp["q"], inp["k"], inp["v"], logits, phi_dev, cfg, return_info=True)
    T = inp["q"].shape[2]
    pos = O.sample_positions(T, rows, c["l"], c["w"], c["l_prime"], c["n"], seed=1)
    got = {k_: info[k_][:, :, pos.to(info[k_].device)].float().cpu() for k_ in ("o_cmp", "o_slc", "o_win")}
    idx = info["indices"][:, :, pos.to(info["indices"].device)].cpu().long()
    del info
    k, v = inp["k"].float().cpu(), inp["v"].float().cpu()
    phi = O.PhiParams(*(params[n_].detach().float().cpu() for n_ in ("pos_embed", "w1", "b1", "w2", "b2")))
    k_cmp, v_cmp, be, _ = O.compress_tokens(k.transpose(-1, -2), v, phi, c["l"], c["d"])
    qr = inp["q"][:, :, pos.to(inp["q"].device)].float().cpu()
    scale = c["dk"] ** -0.5
    idx_ref, agg = O.score_rows(qr, pos, k_cmp, be, l=c["l"], d=c["d"], l_prime=c["l_prime"], n=c["n"], scale=scale)
    amb = O.ambiguous_rows(agg, c["n"])
    mism = (idx != idx_ref).any(-1)
    ref = O.branch_rows(qr, pos, k, v, k_cmp, v_cmp, be, idx, w=c["w"], l_prime=c["l_prime"], scale=scale)
    errs = {n_: round((got[n_] - r_).abs().max().item(), 5) for n_, r_ in zip(("o_cmp", "o_slc", "o_win"), ref)}
    return dict(checked="oracle (CPU, fp32) on sampled query rows of the timed workload", rows=int(mism.numel()),
                ambiguous_rows=int(amb.sum()), mismatched_rows=int(mism.sum()),
                mismatched_outside_ambiguity=int((mism & ~amb).sum()), max_abs=errs, bound_bf16=2e-2)


def cpu_reference_tokens_per_s(T_sample, steps, threads):
    """The reference project's own module (NSAAttention in eval mode: its CPU path through nsa/reference.py, float64
    loops over batch, head and token), forward + backward, from the copy oracle/install_reference.py made."""
    import importlib.util
    root = os.path.join(ROOT, "baseline", "_ref", "nsa")
    if not os.path.exists(os.path.join(root, "kernels.py")):
        raise FileNotFoundError("baseline/_ref/nsa is missing: run oracle/install_reference.py --reference <checkout>")
    if "nsa_reference_project" not in sys.modules:
        spec = importlib.util.spec_from_file_location("nsa_reference_project", os.path.join(root, "__init__.py"),
                                                      submodule_search_locations=[root])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["nsa_reference_project"] = mod
        spec.loader.exec_module(mod)
    R = sys.modules["nsa_reference_project"]
    c = CFG
    torch.set_num_threads(threads)
    torch.manual_seed(0)
    cfg = R.NSAConfig(d_model=c["d_model"], head_dim_qk=c["dk"], head_dim_v=c["dv"], l=c["l"], d=c["d"], l_prime=c["l_prime"], n=c["n"],
                      w=c["w"], n_heads=c["H"], n_kv_groups=c["G"])
    model = R.NSAAttention(cfg).eval()
    times = []
    for _ in range(steps):
        x = torch.randn(1, T_sample, c["d_model"], requires_grad=True)
        t0 = time.perf_counter()
        y, _info = model(x)
        y.backward(torch.ones_like(y))
        times.append(time.perf_counter() - t0)
    return T_sample / (sum(times) / len(times)), sum(times) / len(times)


def run_reference(args):
    """`--impl reference`: the reference's algorithm on the host CPU.  Default: the committed CPU oracle, a vectorised
    port that is some 40 times faster per token than the reference's own Python loops, on a T=4096 sample (kind "port": the
    ratio against it understates the speed-up).  `--cpu-kind reference`: the reference project's own module from
    baseline/_ref on a sample short enough for its loops (kind "reference")."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    T_sample = args.cpu_sample
    if args.cpu_kind == "reference":
        T_sample = min(T_sample, 128)
        if args.warmup > 0:
            cpu_reference_tokens_per_s(T_sample, 1, threads)
        tps, sec = cpu_reference_tokens_per_s(T_sample, max(1, args.steps), threads)
        sample = (f"the reference's NSAAttention (eval: its float64 CPU path) forward + backward, projections included, one sequence "
                  f"of T={T_sample} (same heads/dims as the workload)")
        line = dict(metric=METRIC, value=tps, unit="tokens/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                    ms_per_step=sec * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f64", data="synthetic",
                    impl="reference", config=dict(workload=f"NSA layer fwd+bwd, B=1 per GPU, T={T_sample} sample of T={args.T}", **CFG),
                    cpu_baseline=dict(value=tps, unit="tokens/s", cores=threads, kind="reference", sample=sample),
                    e2e=dict(value=tps, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
        print(json.dumps(line))
        return
    for _ in range(min(args.warmup, 1)):
        cpu_oracle_tokens_per_s(T_sample, 1, threads)
    tps, sec = cpu_oracle_tokens_per_s(T_sample, max(1, args.steps), threads)
    value = tps                 # one host: N sequences take N times as long, so the rate does not grow with --gpus
    sample = f"full layer fwd+bwd, fp32 on bf16-rounded inputs, one sequence of T={T_sample} (same heads/dims as the workload)"
    line = dict(metric=METRIC, value=value, unit="tokens/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=sec * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                impl="reference", config=dict(workload=f"NSA layer fwd+bwd, B=1 per GPU, T={T_sample} sample of T={args.T}", **CFG),
                cpu_baseline=dict(value=value, unit="tokens/s", cores=threads, kind="port", sample=sample),
                e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------

def run_decode(args):
    """Single-token forward steps of one layer against a KV + compressed-KV cache of --T tokens (batch 1)."""
    import nsa
    from nsa.incremental import NSACache, nsa_layer_incremental
    from nsa._lib import lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    c, T, N = CFG, args.T, args.decode
    cfg = nsa.NSAConfig(d_model=c["d_model"], head_dim_qk=c["dk"], head_dim_v=c["dv"], l=c["l"], d=c["d"], l_prime=c["l_prime"],
                        n=c["n"], w=c["w"], n_heads=c["H"], n_kv_groups=c["G"])
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *sh, std=1.0: torch.randn(*sh, generator=g, device=dev) * std
    H, G, dk, dv, l = c["H"], c["G"], c["dk"], c["dv"], c["l"]
    phi = (rn(l, l, std=0.02), rn(2 * dk, dk + l, std=0.02), torch.zeros(2 * dk, device=dev), rn(dk, 2 * dk, std=0.02),
           torch.zeros(dk, device=dev))
    warm = max(args.warmup, 3)
    cache = NSACache(cfg, 1, T, dev, shared_kv=True)
    pre = T - N - warm
    cache.append(phi, rn(1, G, dk, pre).bfloat16(), rn(1, G, pre, dv).bfloat16())
    toks = [(rn(1, G, dk, 1).bfloat16(), rn(1, G, 1, dv).bfloat16(), rn(1, H, 1, dk).bfloat16(), rn(1, 1, 3 * H))
            for _ in range(N + warm)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i, (kn, vn, qn, lg) in enumerate(toks):
        if i == warm:
            torch.cuda.synchronize()
            e0.record()
        cache.append(phi, kn, vn)
        out = nsa_layer_incremental(qn, lg, cache)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / N
    print(json.dumps(dict(metric="NSA layer decode step (cache append + one-token forward), ms per token", value=round(ms, 4),
                          unit="ms", n_gpus=1, steps=N, warmup=warm, higher_is_better=False, dtype="bf16", data="synthetic",
                          config=dict(workload=f"one layer, batch 1, cache of {T} tokens", **c),
                          checksum=float(out.float().sum()), device_timeouts=lib.nsa_device_timeouts(0))))


def run_reference_shape(args):
    """The one shape the reference project times itself (tests/test_large_scale.py:24-32: B=4, H=32, G=8, T=2048, dk=dv=128,
    window 256, sliding-window forward + backward; tokens/s = B*T / (t_fwd + t_bwd)), through this library with CUDA
    events: fp32 tensors (what that test passes; they run on the stride-generic kernels) and bf16 tensors (tensor-core
    kernels)."""
    from nsa import ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, H, G, T, d, w = 4, 32, 8, 2048, 128, 256
    scale = d ** -0.5
    res = {}
    for name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        g = torch.Generator(device=dev).manual_seed(0)
        q, k, v, do = (torch.randn(*s_, generator=g, device=dev).to(dt) for s_ in
                       [(B, H, T, d), (B, G, d, T), (B, G, T, d), (B, H, T, d)])
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        fw, bw = [], []
        for i in range(3 + 10):
            ev[0].record()
            o, L, M = ops.sliding_fwd(q, k, v, w, scale)
            ev[1].record()
            ops.sliding_bwd(q, k, v, o, do, L, M, w, scale)
            ev[2].record()
            torch.cuda.synchronize()
            if i >= 3:
                fw.append(ev[0].elapsed_time(ev[1]))
                bw.append(ev[1].elapsed_time(ev[2]))
        f_ms, b_ms = sorted(fw)[len(fw) // 2], sorted(bw)[len(bw) // 2]
        res[name] = dict(fwd_ms=round(f_ms, 3), bwd_ms=round(b_ms, 3), tokens_per_s=round(B * T / ((f_ms + b_ms) * 1e-3), 1))
    print(json.dumps(dict(metric="sliding-window fwd+bwd at the reference's large-scale test shape", unit="tokens/s",
                          config=dict(workload="B=4 H=32 G=8 T=2048 dk=dv=128 window=256, median of 10 after 3 warm-up"), **res)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--T", type=int, default=65536)
    ap.add_argument("--cpu-sample", type=int, default=4096, help="sequence length of the CPU-oracle sample")
    ap.add_argument("--cpu-kind", default="port", choices=["port", "reference"],
                    help="--impl reference: time the committed CPU oracle (port, default) or the reference project's own module")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-long-context", action="store_true",
                    help="multi-GPU runs: skip the extra leg that times ONE sequence split by position over the GPUs")
    ap.add_argument("--long-context-2t", action="store_true",
                    help="multi-GPU runs: also time the long-context leg at twice --T (always done on 8 GPUs)")
    ap.add_argument("--no-parity", action="store_true", help="skip the sampled-row check of the workload against the oracle")
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the end-to-end leg (default: max(50, --steps))")
    ap.add_argument("--shard", default="sequence", choices=["sequence", "query"],
                    help="sequence: one T-token sequence per GPU (weak scaling, the default); query: ONE T-token sequence "
                         "split by position over the GPUs, K/V all-gathered (long-context mode, strong scaling)")
    ap.add_argument("--decode", type=int, default=0, metavar="N",
                    help="instead of the training step: time N single-token forward steps of one layer against a cache of "
                         "--T tokens (nsa.incremental) and print their own JSON line")
    ap.add_argument("--ref-shape", action="store_true",
                    help="instead of the training step: time the sliding-window branch at the shape the reference's own "
                         "tests/test_large_scale.py times, fp32 and bf16")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.ref_shape:
        return run_reference_shape(args)
    if args.decode > 0:
        return run_decode(args)

    import nsa
    from nsa import _lib
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    T = args.T
    c = CFG
    cfg = nsa.NSAConfig(d_model=c["d_model"], head_dim_qk=c["dk"], head_dim_v=c["dv"], l=c["l"], d=c["d"], l_prime=c["l_prime"],
                        n=c["n"], w=c["w"], n_heads=c["H"], n_kv_groups=c["G"])
    query_mode = args.shard == "query" and world > 1
    if query_mode:
        from nsa.sharding import balanced_query_bounds
        inp, params = make_device_inputs(T, dev, seed=0)        # the same sequence on every rank; each keeps its slice
        # slices sized for equal attention work: w + n*l' keys per query everywhere, plus t/d compressed keys
        bounds = balanced_query_bounds(T, world, POSITION_INDEPENDENT_COST, c["d"])
        t0, t1 = bounds[rank], bounds[rank + 1]
        inp = dict(q=inp["q"][:, :, t0:t1].contiguous(), k=inp["k"][..., t0:t1].contiguous(), v=inp["v"][:, :, t0:t1].contiguous(),
                   do=inp["do"][:, :, t0:t1].contiguous(), x=inp["x"][:, t0:t1].contiguous(), bounds=bounds)
        torch.cuda.empty_cache()
    else:
        inp, params = make_device_inputs(T, dev, seed=rank)
    step_fn = layer_step_query_sharded if query_mode else layer_step
    seqs = 1 if query_mode else world                            # sequences processed per step by the whole job

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput -------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step_fn(inp, params, cfg, world)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_fn(inp, params, cfg, world)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    t_ms = torch.tensor([ms], device=dev)
    if world > 1:
        torch.distributed.all_reduce(t_ms, op=torch.distributed.ReduceOp.MAX)
    ms_per_step = t_ms.item() / args.steps
    value = seqs * T / (ms_per_step * 1e-3)

    # ---- end to end: inputs come from pinned host memory every step, result read back -----------
    host = {k_: torch.empty(v_.shape, dtype=v_.dtype, pin_memory=True).copy_(v_) for k_, v_ in inp.items() if torch.is_tensor(v_)}
    h2d = sum(t_.numel() * t_.element_size() for t_ in host.values())
    res_host = torch.empty(1, dtype=torch.float32, pin_memory=True)

    # Inputs are double-buffered on the device: the copy of step i+1 runs on its own stream while step i computes, as a
    # data loader would feed the layer.  Every step's inputs are copied, and its result read back, inside the timed region.
    copy_stream = torch.cuda.Stream(device=dev)
    slots = [{k_: (torch.empty_like(v_) if torch.is_tensor(v_) else v_) for k_, v_ in inp.items()} for _ in range(2)]
    copied_fwd = [torch.cuda.Event() for _ in range(2)]     # q, k, v, x of the slot have landed
    copied_all = [torch.cuda.Event() for _ in range(2)]     # ... and the upstream gradient dO, first used by the backward
    consumed = [torch.cuda.Event() for _ in range(2)]
    fwd_names = [k_ for k_ in host if k_ != "do"]

    def upload(i):
        with torch.cuda.stream(copy_stream):
            if i >= 2:
                copy_stream.wait_event(consumed[i % 2])
            for k_ in fwd_names:
                slots[i % 2][k_].copy_(host[k_], non_blocking=True)
            copied_fwd[i % 2].record(copy_stream)
            slots[i % 2]["do"].copy_(host["do"], non_blocking=True)
            copied_all[i % 2].record(copy_stream)

    def e2e_run(n):
        cur = torch.cuda.current_stream()
        upload(0)
        for i in range(n):
            if i + 1 < n:
                upload(i + 1)
            cur.wait_event(copied_fwd[i % 2])
            res = step_fn(slots[i % 2], params, cfg, world, before_backward=lambda: cur.wait_event(copied_all[i % 2]))
            res_host.copy_(res.reshape(1), non_blocking=True)
            consumed[i % 2].record(cur)
        cur.synchronize()

    e2e_run(1)
    barrier()
    # The first step's copy (58 ms for 3.19 GB over PCIe) has nothing to hide behind (pipeline fill) and is inside the
    # timed region; 50 steps make the figure the sustained rate of the double-buffered loop (the fill adds 1.2 ms per step
    # to the average) rather than that of its first step.
    e2e_steps = args.e2e_steps if args.e2e_steps > 0 else max(50, args.steps)
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    barrier()
    t_e2e = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        torch.distributed.all_reduce(t_e2e, op=torch.distributed.ReduceOp.MAX)
    e2e_value = seqs * T / (t_e2e.item() / e2e_steps * 1e-3)

    # ---- long-context mode (one sequence split by position), recorded with every multi-GPU run --
    long_context = None
    if world > 1 and not query_mode and not args.no_long_context:
        del inp, host, slots            # the weak-scaling inputs make room; rebuilt below for the profiled step
        torch.cuda.empty_cache()
        long_context = [long_context_leg(args, cfg, dev, world, rank, T, ms_per_step)]
        if world >= 8 or args.long_context_2t:
            long_context.append(long_context_leg(args, cfg, dev, world, rank, 2 * T, ms_per_step))
        torch.cuda.empty_cache()
        inp, _ = make_device_inputs(T, dev, seed=rank)

    # ---- per-kernel times (CUDA events around every launch, outside the timed region) -----------
    prof = _lib.profile_kernels(lambda: step_fn(inp, params, cfg, world))
    launches = sum(n_ for n_, _ in prof.values())
    kflops = kernel_flops(T)
    peaks = measured_peaks()
    timeouts = _lib.lib.nsa_device_timeouts(0)
    if rank == 0:
        cand = {k_: v_ for k_, v_ in prof.items() if k_ in kflops}
        top = max(cand, key=lambda k_: cand[k_][1]) if cand else None
        roofline = None
        if top and not query_mode:   # per-launch FLOP figures assume a whole sequence per launch
            n_l, tot = cand[top]
            achieved = kflops[top] / (tot / n_l * 1e-3) / 1e12
            units = c["G"] * T * c["n"]                                   # (group, query, slot) triples of one launch
            traffic = int(NCU_DRAM_BYTES_PER_UNIT[top] * units) if top in NCU_DRAM_BYTES_PER_UNIT else None
            # `bound` says what limits the kernel.  The dense kernels keep the tensor pipe busiest (ncu, profiles/) and are
            # rated by FLOPs against the sustained cuBLAS rate.  The selection kernels move 16 KB (backward) / 10 KB (forward)
            # through HBM per 13.6 / 5.2 MFLOP unit and are rated by their algorithmic bytes against the measured copy
            # bandwidth: bringing rows into L2 earlier makes the backward slower, not faster (profiles/).
            if top in NCU_DRAM_BYTES_PER_UNIT:
                gbs = selection_bytes_per_unit(top) * units / (tot / n_l * 1e-3) / 1e9
                roofline = dict(bound="hbm", kernel=top, achieved=round(gbs, 1), peak=peaks["hbm_gbs"], unit="GB/s",
                                frac=round(gbs / peaks["hbm_gbs"], 4), traffic=traffic,
                                counters="dram 51 % busy, tensor pipe 33 % (ncu, T=8192, where 56 % of the gathers hit L2)",
                                traffic_source="ncu dram bytes at T=8192 scaled by (group, query, slot) units; lower bound",
                                peak_source=peaks["source"] + " (copy bandwidth)", tflops=round(achieved, 1),
                                ms_per_launch=round(tot / n_l, 4))
            else:
                roofline = dict(bound="tensor", kernel=top, achieved=round(achieved, 1), peak=peaks["tflops_sustained"],
                                unit="TFLOP/s", frac=round(achieved / peaks["tflops_sustained"], 4), traffic=None,
                                counters="tensor pipe busiest (ncu, T=8192)", traffic_source=None,
                                peak_source=peaks["source"] + " (sustained bf16)", ms_per_launch=round(tot / n_l, 4))
        att = attention_flops(T)
        att_total = sum(att[b_][p_] for b_ in att for p_ in att[b_])
        kern_ms = sum(ms_ for _, ms_ in prof.values())
        breakdown = {k_: round(v_[1], 3) for k_, v_ in sorted(prof.items(), key=lambda kv: -kv[1][1])}
        cpu = None
        if not args.no_cpu:
            threads = os.cpu_count() or 1
            tps, sec = cpu_oracle_tokens_per_s(args.cpu_sample, 1, threads)
            cpu = dict(value=round(tps, 2), unit="tokens/s", cores=threads, kind="port",
                       sample=f"one full-layer fwd+bwd of the CPU oracle (fp32) at T={args.cpu_sample}, same heads/dims, {sec:.1f} s")
        parity = None
        if not args.no_parity and not query_mode:
            parity = sampled_parity(inp, params, cfg)
        line = dict(metric=METRIC, value=round(value, 1), unit="tokens/s", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
                    ms_per_step=round(ms_per_step, 3), higher_is_better=True, scaling="strong" if query_mode else "weak",
                    vs_baseline=None, dtype="bf16",
                    data="synthetic", impl="ours",
                    config=dict(workload=(f"NSA layer fwd+bwd, ONE sequence of T={T} split by position over the GPUs, K/V all-gathered"
                                          if query_mode else f"NSA layer fwd+bwd, one sequence per GPU, T={T}"),
                                l2="inputs (>= 1.6 GB per tensor) exceed the 126 MB L2",
                                parallelism=f"sp{world}" if query_mode else f"dp{world}", **c),
                    e2e=dict(value=round(e2e_value, 1), unit="tokens/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=4, steps=e2e_steps),
                    gpu_launches=launches * args.steps, roofline=roofline, cpu_baseline=cpu, clocks=clocks,
                    attention_tflops_per_s=round(att_total / (ms_per_step * 1e-3) / 1e12, 1),
                    attention_frac_of_peak=round(att_total / (ms_per_step * 1e-3) / 1e12 / peaks["tflops_sustained"] / (world if query_mode else 1), 4),
                    kernel_ms=breakdown, kernel_ms_total=round(kern_ms, 3), device_timeouts=timeouts, parity=parity,
                    long_context=long_context)
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
