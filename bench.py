"""Decode throughput of the 'cuda fp16i8' path at the RWKV-4 7B shape, one JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Workload (N = 1 and every rank at N > 1): RWKV-4 7B-shape model (32 x 4096, ffn 16384,
vocab 50277), seeded random-init weights packed to uint8 on the GPU, a 1024-token seeded
prompt, then greedy decoding.  One "step" = one decoded token.  Ranks are independent
streams (token seed 2000 + rank), no collective on the data path: weak scaling.

  value     tokens/s over all ranks; token ids stay on the device (argmax -> next forward).
  e2e       the same loop through RWKV.forward([int], state) with HOST token ids in and the
            fp32 logits copied to pinned host memory out, host-side argmax.
  roofline  mm8_one GEMV launches of a decode step timed one by one with CUDA events:
            algorithmic bytes / time, against the measured HBM copy bandwidth.
  cpu_baseline  the reference's CPU arithmetic for the same matmuls (dequantise, then fp32
            matmul) timed on the host cores over a bounded sample, scaled to a whole token.

--impl reference runs only that CPU arm (rank 0), printing the same line shape.
"""
from __future__ import annotations

import argparse
import copy as _copy
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = "v4-7b"
PROMPT = 1024
METRIC = "fp16i8_decode_tokens_per_s_rwkv4_7b_shape"


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU arithmetic for mm8 (dequantise the matrix, then fp32 matmul),
# restated in oracle/rwkv_oracle.py::mm8_spec, on a bounded sample of a 7B-shape token.
# ------------------------------------------------------------------------------------------
def matrices_of_token(shape):
    import chatrwkv_b200.synth as synth
    L, D, Fn, V = synth.SHAPES[shape]
    per_layer = [(D, D)] * 4 + [(D, D), (D, Fn), (Fn, D)]
    return L, per_layer, (D, V)


def cpu_sample_setup(N, M):
    import torch
    g = torch.Generator().manual_seed(3000)
    w = torch.randint(0, 256, (N, M), dtype=torch.uint8, generator=g)
    mx = torch.randn(M, generator=g) * 0.01
    rx = torch.rand(M, generator=g) * 0.01
    my = torch.randn(N, 1, generator=g) * 0.01
    ry = torch.rand(N, 1, generator=g) * 0.01
    x = torch.randn(N, generator=g)
    return x, w, mx, rx, my, ry


def cpu_arm(steps, warmup, budget_s=100.0):
    """Times mm8_spec on (4096, 4096) matrices -- the cost is proportional to the number of
    weight bytes -- and scales to the 7,185,256,448 weight bytes of one 7B-shape token."""
    import torch
    from oracle import rwkv_oracle as orc
    # all host threads, also under torchrun (which exports OMP_NUM_THREADS=1 to its workers)
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        torch.set_num_threads(os.cpu_count() or 1)
    L, per_layer, head = matrices_of_token(WORKLOAD)
    token_bytes = L * sum(n * m for n, m in per_layer) + head[0] * head[1]
    N = M = per_layer[0][0]
    args = cpu_sample_setup(N, M)
    t0 = time.perf_counter()
    orc.mm8_spec(*args)
    t_one = time.perf_counter() - t0
    total = max(1, steps + warmup)
    reps = max(1, min(8, int(budget_s / (t_one * total))))      # matrices per step
    for _ in range(warmup):
        for _ in range(reps):
            orc.mm8_spec(*args)
    t0 = time.perf_counter()
    for _ in range(steps):
        for _ in range(reps):
            orc.mm8_spec(*args)
    dt = time.perf_counter() - t0
    bytes_done = steps * reps * N * M
    tok_s = (bytes_done / dt) / token_bytes
    return {"value": tok_s, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{steps} steps x {reps} mm8 (dequantise + fp32 matmul) of {N}x{M} uint8, scaled by weight "
                      f"bytes to a {token_bytes}-byte token", "ms_per_step": dt / steps * 1e3,
            "host_cpus": os.cpu_count()}


# ------------------------------------------------------------------------------------------
def reference_cpu_arm(mode, steps, warmup, shape=WORKLOAD, timeout=900):
    """The reference's own 'cpu fp32i8' runtime in a child process (oracle/ref_cpu_bench.py); None when the
    staged runtime is missing or the child fails."""
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "pkg", "rwkv", "model.py")):
        return None
    env = dict(os.environ)
    env.pop("OMP_NUM_THREADS", None)            # torchrun exports 1; the CPU arm uses all host threads
    cmd = [sys.executable, "-m", "oracle.ref_cpu_bench", mode, "--steps", str(steps), "--warmup", str(warmup), "--shape", shape]
    try:
        r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
        if r.returncode != 0:
            return None
        out = json.loads(r.stdout.strip().splitlines()[-1])
        out["host_cpus"] = os.cpu_count()
        return out
    except Exception:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--shape", default=WORKLOAD)
    ap.add_argument("--prompt", type=int, default=PROMPT)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shard", action="store_true",
                    help="second multi-GPU mode: ONE model, every packed matrix split by output columns over the "
                         "ranks with an exchange after each matmul (strong scaling; use with --shape v4-14b)")
    ap.add_argument("--sweep", action="store_true",
                    help="operator sweep instead of the model bench: mm8_one (T=1) and mm8_seq (T=16,128,1024) on the "
                         "four (N, M) shapes of the task's operator config; one JSON line with a 'sweep' list")
    ap.add_argument("--sequences", type=int, default=0,
                    help="S independent sequences dealt to the ranks (s mod N), each with its own prefill of --prompt "
                         "tokens and --steps greedy tokens; value = decoded tokens of all sequences / time")
    ap.add_argument("--sweep-part", default="all", choices=["all", "mm8", "wkv"], help="with --sweep: which operators")
    ap.add_argument("--sweep-T", type=int, default=0, help="with --sweep: only this row / step count")
    ap.add_argument("--batch", type=int, default=0,
                    help="batched decode: B sequences per GPU advance one token per step through RWKV.forward_batch; "
                         "value = B x GPUs x steps / time")
    ap.add_argument("--layers", type=int, default=0,
                    help="profiling aid: build only this many layers of the shape (the line is then not a bench result)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    metric = METRIC if a.shape == WORKLOAD else f"fp16i8_decode_tokens_per_s_rwkv{a.shape.replace('-', '_')}_shape"

    if a.impl == "reference":
        if rank != 0:
            return
        k = max(1, min(a.steps, 6))             # bounded: a step costs ~8 s of host time at the 7B width
        cb = reference_cpu_arm("token7b", k, min(a.warmup, 1), a.shape) or cpu_arm(a.steps, a.warmup)
        line = {"impl": "reference", "metric": metric, "value": cb["value"], "unit": "tokens/s", "n_gpus": a.gpus,
                "steps": a.steps, "warmup": a.warmup, "ms_per_step": cb["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"rwkv{a.shape} shape 'cpu fp32i8' greedy decode, batch 1, on the host cores; "
                                       f"bounded sample: {cb['sample']}"},
                "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    import torch
    import torch.distributed as dist
    from chatrwkv_b200 import shard, synth
    from chatrwkv_b200.model import RWKV

    if a.sweep:
        if rank == 0:
            print(json.dumps(operator_sweep(torch.device("cuda", local_rank), part=a.sweep_part, only_T=a.sweep_T)), flush=True)
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    L, D, Fn, V = synth.SHAPES[a.shape]
    if a.layers > 0:
        L = a.layers
    version = 6 if a.shape.startswith("v6") else 4
    ck = synth.make_checkpoint(version, L, D, Fn, V, seed=1002, device=dev)
    sharded = a.shard and world > 1
    model = RWKV(ck, f"cuda:{local_rank} fp16i8", verbose=False,
                 shard_rank=rank if sharded else 0, shard_world=world if sharded else 1)
    del ck
    torch.cuda.empty_cache()

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    weight_gb = sum(t.numel() for t in model.w.values() if torch.is_tensor(t) and t.dtype == torch.uint8) / 1e9
    n_mm = L * (7 if version == 4 else 8) + 1

    def decode_loop(tok, state, n):
        for _ in range(n):
            logits, state = model.forward(tok, state)
            tok = torch.argmax(logits).reshape(1)
        return tok, state

    if a.batch > 0 and a.sequences == 0:
        # ---- batched decode: B sequences per GPU, one token each per step, no prefill (zero states) ----
        B = a.batch
        tok = torch.tensor(synth.make_tokens(B, V, 2000 + rank), dtype=torch.int64, device=dev)
        logits, bstate = model.forward_batch(tok, None)
        for _ in range(a.warmup):
            logits, bstate = model.forward_batch(torch.argmax(logits, dim=-1), bstate)
        sampler = ClockSampler(local_rank)
        barrier()
        sampler.start()
        ev0.record()
        for _ in range(a.steps):
            logits, bstate = model.forward_batch(torch.argmax(logits, dim=-1), bstate)
        ev1.record()
        barrier()
        clocks = sampler.stop()
        ms = ev0.elapsed_time(ev1)
        times = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        ms = times.item()
        if rank == 0:
            line = {"metric": metric.replace("decode_tokens", f"batch{B}_decode_tokens"), "unit": "tokens/s", "n_gpus": world,
                    "value": world * B * a.steps / (ms / 1e3), "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
                    "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                    "config": {"workload": f"rwkv{a.shape} shape 'cuda fp16i8': {B} independent sequences per GPU decoded one token "
                                           f"per step together (RWKV.forward_batch), greedy, from empty states",
                               "parallelism": "independent batches, one per GPU, no collective",
                               "l2": f"inputs larger than L2 ({weight_gb:.2f} GB of packed weights streamed per step)"},
                    "per_sequence_tokens_per_s": a.steps / (ms / 1e3), "clocks": clocks, "graph": bool(model._use_graph)}
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    if a.sequences > 0:
        # ---- S independent sequences over the ranks, each prefill + greedy decode, one after the other ----
        mine = shard.assign_sequences(a.sequences, world, rank)
        model.forward(synth.make_tokens(min(a.prompt, 192), V, 1), None)            # untimed: sizes workspaces
        _, st = model.forward(synth.make_tokens(8, V, 1), None)
        decode_loop(torch.zeros(1, dtype=torch.int64, device=dev), st, a.warmup)     # untimed: captures the decode graphs
        sampler = ClockSampler(local_rank)
        barrier()
        sampler.start()
        ev0.record()
        pre_ms = 0.0
        if a.batch > 0:
            # prefill one by one, then groups of --batch sequences decode together (RWKV.forward_batch)
            import copy
            for g0 in range(0, len(mine), a.batch):
                group = mine[g0:g0 + a.batch]
                p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                p0.record()
                states, first = [], []
                for sq in group:
                    logits, state = model.forward(synth.make_tokens(a.prompt, V, 2000 + sq), None)
                    states.append(state)
                    first.append(torch.argmax(logits).reshape(1))
                bstate = model.stack_states(states)
                p1.record()
                tok = torch.cat(first)
                for _ in range(a.steps):
                    logits, bstate = model.forward_batch(tok, bstate)
                    tok = torch.argmax(logits, dim=-1)
                torch.cuda.synchronize(dev)
                pre_ms += p0.elapsed_time(p1)
            mine_iter = []
        else:
            mine_iter = mine
        for sq in mine_iter:
            prompt = synth.make_tokens(a.prompt, V, 2000 + sq)
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            p0.record()
            logits, state = model.forward(prompt, None)
            p1.record()
            decode_loop(torch.argmax(logits).reshape(1), state, a.steps)
            torch.cuda.synchronize(dev)
            pre_ms += p0.elapsed_time(p1)
        ev1.record()
        barrier()
        clocks = sampler.stop()
        total_ms = ev0.elapsed_time(ev1)
        times = torch.tensor([total_ms, pre_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        total_ms, pre_ms = times.tolist()
        if rank == 0:
            dec_tokens = a.sequences * a.steps
            line = {"metric": metric.replace("decode_tokens", "sequences_decode_tokens"), "unit": "tokens/s", "n_gpus": world,
                    "value": dec_tokens / ((total_ms - pre_ms) / 1e3), "steps": a.steps, "warmup": a.warmup,
                    "ms_per_step": (total_ms - pre_ms) / (a.steps * max(1, -(-len(mine) // a.batch) if a.batch > 0 else len(mine))),
                    "higher_is_better": True,
                    "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                    "config": {"workload": f"rwkv{a.shape} shape 'cuda fp16i8': {a.sequences} independent sequences dealt to "
                                           f"{world} GPU(s) (s mod N), each a {a.prompt}-token prefill then {a.steps} greedy "
                                           f"tokens; " + (f"prefill one by one, decode in batches of {a.batch} (forward_batch)"
                                                           if a.batch > 0 else "one sequence at a time per GPU"),
                               "parallelism": "independent sequences, no collective",
                               "l2": f"inputs larger than L2 ({weight_gb:.2f} GB of packed weights streamed per step)"},
                    "whole_job": {"seconds": total_ms / 1e3, "prefill_seconds_max_rank": pre_ms / 1e3,
                                  "prefill_tokens": a.sequences * a.prompt, "decoded_tokens": dec_tokens,
                                  "all_tokens_per_s": a.sequences * (a.prompt + a.steps) / (total_ms / 1e3)},
                    "gpu_launches": None, "clocks": clocks, "graph": bool(model._use_graph),
                    "decode_path": model.decode_path()}
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    prompt = synth.make_tokens(a.prompt, V, 2000 + (0 if sharded else rank))
    # ---- prefill (reported, not the headline) ------------------------------------------
    model.forward(prompt[:192], None)            # untimed: sizes workspaces, loads kernels
    prefill_ms = float("inf")
    for _ in range(2):                            # the first full-length call also sizes the operator workspaces
        torch.cuda.synchronize(dev)
        ev0.record()
        logits, state = model.forward(prompt, None)
        ev1.record()
        torch.cuda.synchronize(dev)
        prefill_ms = min(prefill_ms, ev0.elapsed_time(ev1))

    # ---- device-resident greedy decode --------------------------------------------------
    tok = torch.argmax(logits).reshape(1)
    tok, state = decode_loop(tok, state, a.warmup)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    torch.cuda.cudart().cudaProfilerStart()      # lets `ncu --profile-from-start off` see the timed region only
    ev0.record()
    tok, state = decode_loop(tok, state, a.steps)
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)

    # ---- end to end: host token in, logits to pinned host memory, host argmax ----------
    host_logits = torch.empty(V, dtype=torch.float32).pin_memory()
    t_host = int(tok.item())
    for _ in range(a.warmup):
        logits, state = model.forward([t_host], state)
        host_logits.copy_(logits, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
        t_host = int(host_logits.argmax())
    barrier()
    ev0.record()
    for _ in range(a.steps):
        logits, state = model.forward([t_host], state)
        host_logits.copy_(logits, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
        t_host = int(host_logits.argmax())
    ev1.record()
    barrier()
    torch.cuda.cudart().cudaProfilerStop()
    clocks = sampler.stop()
    e2e_ms = ev0.elapsed_time(ev1)

    times = torch.tensor([dev_ms, e2e_ms, prefill_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, prefill_ms = times.tolist()
    path_default = model.decode_path()
    launches_default = model.launches_per_token()

    # ---- the other decode paths of the runtime, 64 steps each (rank 0, single-GPU mode only) ----
    other = {}
    if rank == 0 and not sharded and a.layers == 0:
        from chatrwkv_b200 import _lib
        n_alt = min(64, a.steps)
        alts = [("launch_per_matmul_fp32_arithmetic", "launch", 8), ("launch_per_matmul_general_kernel", "launch", -1)]
        if version == 4:
            alts.append(("persistent_weight_stream_kernel", "stream", 0))
        for label, path, variant in alts:
            if path == path_default and variant == 0:
                continue
            _lib.lib().rwkv_mm8_one_set_variant(max(variant, 0))
            _lib.lib().rwkv_mm8_one_set_lean(0 if variant < 0 else -1)        # -1 here: mm8_cluster_kernel with the default arithmetic
            model.set_decode_path(path)
            tok, state = decode_loop(tok, state, 4)
            torch.cuda.synchronize(dev)
            ev0.record()
            tok, state = decode_loop(tok, state, n_alt)
            ev1.record()
            torch.cuda.synchronize(dev)
            other[label] = {"tokens_per_s": n_alt / (ev0.elapsed_time(ev1) / 1e3), "steps": n_alt}
            if path == "stream":
                other[label]["wait_error"] = model.stream_error()
        _lib.lib().rwkv_mm8_one_set_variant(0)
        _lib.lib().rwkv_mm8_one_set_lean(-1)
        model.set_decode_path(path_default)
        tok, state = decode_loop(tok, state, 2)

    # ---- generation with the sampler on the device (nucleus sampling, penalties): the loop of PIPELINE.generate
    sampling = None
    if rank == 0 and not sharded and a.layers == 0 and version == 4:
        from chatrwkv_b200.pipeline import PIPELINE, PIPELINE_ARGS
        n_gen = min(64, a.steps)
        pl = PIPELINE(model, seed=1)
        pargs = PIPELINE_ARGS(temperature=1.0, top_p=0.85, top_k=0, alpha_frequency=0.2, alpha_presence=0.2)
        sampling = {"steps": n_gen, "args": "temperature 1.0, top_p 0.85, presence/frequency penalties 0.2 (the reference's defaults)"}
        for label, fn in (("token_stays_on_device", lambda st: pl.generate_tokens([int(tok)], n_gen, pargs, st)),
                          ("token_to_host_every_step", lambda st: (pl.generate([int(tok)], n_gen, pargs, None, st), None))):
            fn(_copy.deepcopy(state))
            torch.cuda.synchronize(dev)
            t0 = time.perf_counter()
            fn(_copy.deepcopy(state))
            torch.cuda.synchronize(dev)
            sampling[label + "_tokens_per_s"] = n_gen / (time.perf_counter() - t0)
        from chatrwkv_b200.pipeline import Sampler
        smp = Sampler(V, dev, pargs, seed=2)
        lg = torch.randn(V, device=dev)
        for _ in range(3):
            smp.sample(lg)
        ev0.record()
        for _ in range(20):
            smp.sample(lg)
        ev1.record()
        torch.cuda.synchronize(dev)
        sampling["sampler_kernel_us"] = ev0.elapsed_time(ev1) / 20 * 1e3

    # ---- roofline of the dominant kernel (rank 0): one decode step of direct launches, event-timed
    roof = None
    if rank == 0:
        roof = None if sharded else gemv_roofline(model, dev)
    cb = None
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        cb = reference_cpu_arm("token7b", 2, 1, a.shape) or cpu_arm(steps=6, warmup=1, budget_s=25.0)
        c0 = reference_cpu_arm("config0", 16, 2)
        if c0 is not None:
            cb["config0"] = c0

    # ---- one RWKV-4 14B-shape model column-sharded over all ranks (peer stores in the matmul epilogue), 64 tokens
    graph_default = bool(model._use_graph)
    sharded_14b = None
    if world > 1 and not sharded and a.layers == 0 and a.shape == WORKLOAD and os.environ.get("RWKV_B200_BENCH_SHARDED", "1") != "0":
        del model, state, logits
        torch.cuda.empty_cache()
        sharded_14b = sharded_14b_decode(dev, local_rank, rank, world, barrier, steps=64)

    if rank == 0:
        line = {
            "metric": metric, "value": (1 if sharded else world) * a.steps / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": dev_ms / a.steps, "higher_is_better": True,
            "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"parallelism": ("one model column-sharded over %d GPUs, exchange after each matmul" % world) if sharded
                                      else "independent streams, one per GPU, no collective",
                       "workload": f"rwkv{a.shape} shape (L={L}, D={D}, ffn={Fn}, vocab={V}) 'cuda fp16i8', batch 1 per "
                                   f"GPU: {a.prompt}-token prefill then greedy decode; one independent stream per GPU",
                       "l2": f"inputs larger than L2 ({weight_gb:.2f} GB of packed weights streamed per step on this rank)",
                       "mm8_matmuls_per_token": n_mm},
            "e2e": {"value": (1 if sharded else world) * a.steps / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 8,
                    "d2h_bytes_per_step": V * 4},
            "gpu_launches": launches_default * a.steps * 2,
            "decode_path": path_default, "graph": graph_default,
            "arithmetic": "x*ry as 30-bit fixed point per vector, exact 64-bit integer sums" if path_default == "stream"
                          else "x*ry as 16-bit fixed point per CTA slice, exact 32-bit integer sums (other_decode_paths: fp32)",
            "other_decode_paths": other, "sampling": sampling,
            "prefill": {"tokens": a.prompt, "ms": prefill_ms, "tokens_per_s": a.prompt / (prefill_ms / 1e3)},
            "clocks": clocks, "roofline": roof, "cpu_baseline": cb,
        }
        if sharded_14b is not None:
            line["sharded_14b"] = sharded_14b
        if a.layers > 0:
            line["note"] = f"profiling run with {a.layers} layers: not a benchmark result"
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def sharded_14b_decode(dev, local_rank, rank, world, barrier, steps=64):
    """Greedy decode of ONE RWKV-4 14B-shape model whose matrices are split by output columns over all ranks
    (every rank streams 1/world of the weights per token; the kernels store their columns into the peers' buffers
    and wait, bounded, on arrival words).  Every rank takes part; returns the record on every rank (max over ranks)."""
    import torch
    import torch.distributed as dist
    from chatrwkv_b200 import synth
    from chatrwkv_b200.model import RWKV
    rec = {"n_gpus": world, "steps": steps, "exchange": "peer stores from the matmul epilogue + arrival words (no collective)"}
    ok = 1
    try:
        L, D, Fn, V = synth.SHAPES["v4-14b"]
        ck = synth.make_checkpoint(4, L, D, Fn, V, seed=1002, device=dev)
        m = RWKV(ck, f"cuda:{local_rank} fp16i8", verbose=False, shard_rank=rank, shard_world=world)
        del ck
        torch.cuda.empty_cache()
        tok = torch.zeros(1, dtype=torch.int64, device=dev)
        st = None
        for _ in range(6):
            lg, st = m.forward(tok, st)
            tok = torch.argmax(lg).reshape(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            lg, st = m.forward(tok, st)
            tok = torch.argmax(lg).reshape(1)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        err = int(m.peer_error())
        graph = bool(m._use_graph)
    except Exception as e:                      # reported, and the other ranks still meet this rank below
        ok, ms, err, graph = 0, 0.0, -1, False
        rec["error"] = f"{type(e).__name__}: {e}"[:200]
    t = torch.tensor([ms, float(err != 0), float(1 - ok)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, any_err, any_fail = t.tolist()
    if any_fail:
        rec.setdefault("error", "another rank failed")
        return rec
    rec.update({"tok_s": steps / (ms / 1e3), "ms_per_step": ms / steps, "wait_ran_out": bool(any_err), "graph": graph,
                "shape": "rwkv v4-14b (L=40, D=5120, ffn=20480)"})
    return rec


def operator_sweep(dev, iters=24, part="all", only_T=0):
    """mm8_one / mm8_seq through torch.ops.rwkv on seeded inputs (weights N(0, 0.02) packed on the GPU,
    activations N(0, 1)), each timed as a CUDA graph of `iters` calls that cycle through enough
    distinct packed matrices to exceed L2 several times over; CUDA events around 3 replays."""
    import torch
    from chatrwkv_b200 import ops
    torch.cuda.set_device(dev)
    peak, how = measured_peaks()
    out = []
    for (N, M) in ([(4096, 4096), (4096, 16384), (16384, 4096), (5120, 20480)] if part in ("all", "mm8") else []):
        copies = max(2, int(600e6 // (N * M)) + 1)
        g = torch.Generator(device=dev).manual_seed(3000)
        packs = []
        for _ in range(copies):
            w = (torch.randn(N, M, generator=g, device=dev) * 0.02).half().float()
            packs.append(ops.quantize_weight(w, torch.float16))
            del w
        for T in ((1, 16, 128, 1024) if only_T == 0 else (only_T,)):
            x = torch.randn((T, N) if T > 1 else (N,), generator=g, device=dev).half()
            y = torch.zeros(M, dtype=torch.float32, device=dev) if T == 1 else \
                torch.empty((T, M), dtype=torch.float16, device=dev)

            def call(i):
                q, mx, rx, my, ry = packs[i % copies]
                if T == 1:
                    torch.ops.rwkv.mm8_one(N, M, x, q, mx, rx, my, ry, y)
                else:
                    torch.ops.rwkv.mm8_seq(T, N, M, x, q, mx, rx, my, ry, y)
            side = torch.cuda.Stream(dev)           # operator workspaces are per stream: warm up on the capture stream
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                call(0)
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(iters):
                    call(i)
            graph.replay()
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                graph.replay()
            e1.record()
            torch.cuda.synchronize(dev)
            us = e0.elapsed_time(e1) / (3 * iters) * 1e3
            nbytes = N * M + 2 * T * N + (4 if T == 1 else 2) * T * M + 4 * (N + M)
            out.append({"N": N, "M": M, "T": T, "us": round(us, 2), "GB/s": round(nbytes / us / 1e3, 1),
                        "frac_of_hbm_peak": round(nbytes / us / 1e3 / peak, 3), "TFLOP/s": round(2.0 * T * N * M / us / 1e6, 1)})
        del packs
        torch.cuda.empty_cache()
    # WKV recurrences at the 7B width (C = 4096, 64 heads of 64): fp32 operands as on the model path
    wkv = []
    C, H = 4096, 64
    Nh = C // H
    g = torch.Generator(device=dev).manual_seed(3001)
    for T in (((16, 256, 2048) if only_T == 0 else (only_T,)) if part in ("all", "wkv") else ()):
        k, v, r = (torch.randn(T, C, generator=g, device=dev) for _ in range(3))
        w6 = torch.exp(-torch.exp(torch.rand(T, C, generator=g, device=dev) * 6 - 5))
        w4, u = -torch.exp(torch.rand(C, generator=g, device=dev) * 6 - 5), torch.rand(C, generator=g, device=dev) * 2 - 1
        y = torch.empty(T, C, device=dev)
        aa, bb, pp = torch.zeros(C, device=dev), torch.zeros(C, device=dev), torch.full((C,), -1e30, device=dev)
        S = torch.zeros(H, Nh, Nh, device=dev)
        cases = {
            "wkv_forward (v4)": (lambda: torch.ops.rwkv.wkv_forward(1, T, C, w4, u, k, v, y, aa, bb, pp), 12 * T * C + 32 * C),
            "rwkv5 forward_fp32": (lambda: torch.ops.rwkv5.forward_fp32(1, T, C, H, S, r, k, v, w6[0].contiguous(), u, y),
                                   16 * T * C + 8 * H * Nh * Nh + 8 * C),
            "rwkv6 forward_fp32": (lambda: torch.ops.rwkv6.forward_fp32(1, T, C, H, S, r, k, v, w6, u, y),
                                   20 * T * C + 8 * H * Nh * Nh + 4 * C),
        }
        for name, (fn, nbytes) in cases.items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            torch.cuda.synchronize(dev)
            us = e0.elapsed_time(e1) / 10 * 1e3
            wkv.append({"op": name, "T": T, "C": C, "us": round(us, 1), "GB/s": round(nbytes / us / 1e3, 1),
                        "us_per_token": round(us / T, 3)})
    return {"sweep": out, "wkv": wkv, "hbm_peak_gbs": peak, "peak_source": how,
            "timing": "mm8: CUDA graph of %d calls over distinct matrices; wkv: 10 direct calls" % iters}


def gemv_roofline(model, dev, reps=30):
    """HBM roofline of the decode kernel.  Decode steps are timed with CUDA events on the
    launching stream (token id already on the device) and divided
    into the algorithmic bytes of its mm8_one problems: N*M weight bytes + 6N (x, my, ry) +
    4M (mx, rx) + the output vector, summed over every matmul of the token."""
    import torch
    peak, how = measured_peaks()
    v4 = model.version == 4
    tot_b = 0
    for name, t in model.w.items():         # every packed matrix is read once per token
        if torch.is_tensor(t) and t.dtype == torch.uint8:
            N, M = t.shape
            tot_b += N * M + 6 * N + 4 * M + (4 if name == "head.weight" else 2) * M
    step_fn = model._step_one_v4 if v4 else model._step_one_v56
    path = model.decode_path()
    # the step as the runtime issues it: the captured CUDA graph of a token (embedding row gather + the launches) when
    # graphs are on, else direct launches; a step reads one state set and writes the other, hence the alternation
    graphs = getattr(model, "_graphs", None)
    use_graph = bool(getattr(model, "_use_graph", False)) and graphs is not None and all(g is not None for g in graphs)
    run = (lambda c: graphs[c].replay()) if use_graph else step_fn
    reps += reps & 1
    cur = model._cur
    for _ in range(4):
        run(cur)
        cur ^= 1
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run(cur)
        cur ^= 1
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / reps
    n_launch = 1 if path == "stream" else model.launches_per_token()
    achieved = tot_b / (ms / 1e3) / 1e9
    traffic, source = None, None
    try:
        with open(os.path.join(ROOT, "profiles", "mm8_traffic.json")) as f:
            t = json.load(f)
        key = "stream" if path == "stream" else "launch"
        ratio = t[key]["dram_bytes_per_algorithmic_byte"] if key in t else t["dram_bytes_per_algorithmic_byte"]
        traffic = ratio * tot_b / n_launch
        source = "scaled: DRAM bytes per algorithmic byte from an ncu capture of a 2-layer model of the same shape"
    except Exception:
        pass
    kernel = "mm8_stream_kernel" if path == "stream" else "mm8_lean_kernel"
    return {"bound": "hbm", "kernel": kernel, "achieved": achieved,
            "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": how, "traffic": traffic,
            "traffic_source": source, "launches_per_step": n_launch, "avg_launch_us": ms / n_launch * 1e3,
            "algorithmic_bytes_per_launch": tot_b / n_launch, "frac_of_8000": achieved / 8000.0,
            "timed": "CUDA events around %d replays of the token's CUDA graph" % reps if use_graph else "CUDA events around %d steps of direct launches" % reps,
            "wait_error": model.stream_error() if path == "stream" else 0}


if __name__ == "__main__":
    main()
