"""Benchmark of the fused tensor-parallel epilogue (all-reduce + residual + RMSNorm + FP8).

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...        # the reference's CPU path on the host cores

A step is ONE call of the fused operator on the headline workload, config 3 of the
baseline: per-rank bf16 partial [1024, 8192], residual [1024, 8192], weight [8192],
per-token dynamic FP8-e4m3 (scale = amax / 448).  At one GPU there is no exchange and the
no-communication kernel runs on the same shape.  The message (16 MiB) is smaller than L2, so
the timed loop rotates over enough distinct buffer sets to exceed L2 several times.

Rank 0 prints one JSON line: `value` is microseconds per call with inputs resident in HBM,
timed with CUDA events over exactly K calls (max over ranks); `e2e` is the same call through
the public Python API with the step's inputs copied from pinned host memory and its results
copied back inside the timed region.  `sweep` holds the other configs (decode 8 x 8192 with a
static scale, prefill 16384 x 7168 with outliers, the 32 x 8192 message of the decoder model).
Inputs are seeded synthetic tensors with the distributions of the baseline configs.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 << 20
NVLINK_PEER_COPY_GBS = 770.0      # measured peer copy per direction on this pool (nominal 900)
NVLINK_SM_STORE_GBS = 690.0       # measured here: SM-issued 16-byte peer stores, both directions busy (copy engine: 754)
HBM_FALLBACK_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of the one-GPU kernel per token at hidden 8192, from the
# ncu capture summarised in profiles/ (185.0 MB per launch of 4096 tokens; traffic grows with the tokens)
K1_DRAM_TRAFFIC_BYTES_PER_TOKEN_H8192 = 185.0e6 / 4096


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


def hbm_bytes(tokens, hidden):
    """Algorithmic HBM bytes of one call at one GPU: read x, read residual, write residual_out
    (bf16 each), write FP8, write scales, read weight."""
    return tokens * hidden * (2 + 2 + 2 + 1) + 4 * tokens + 2 * hidden


def bus_bytes(tokens, hidden, n):
    """NVLink bytes per GPU per direction, all-reduce bus-bandwidth convention."""
    return 2.0 * (n - 1) / n * tokens * hidden * 2


# ---------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            # samples under load: the upper half by power draw
            order = sorted(range(len(sm)), key=lambda i: power[i])
            load = order[len(order) // 2:]
            out.update(sm_mhz=statistics.median(sm[i] for i in load), sm_max_mhz=max(smax),
                       reasons=sorted(reasons), samples=len(sm), power_w_max=max(power))
        return out


# ---------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------
def make_sets(cfg, rank, world, nsets, device):
    """`nsets` distinct input/output buffer sets for one config (seeded, config distributions)."""
    from gpuk_b200 import workloads as oin
    sets = []
    w = oin.make_weight(cfg).to(device)
    base_x = oin.make_partial(cfg, rank, world).to(device)
    base_r = oin.make_residual(cfg).to(device)
    for i in range(nsets):
        x = base_x if i == 0 else base_x.roll(i, 0).contiguous()
        r = base_r if i == 0 else base_r.roll(i, 0).contiguous()
        res_out = torch.empty_like(x)
        if cfg.quant_type == 4:
            scale = torch.tensor([cfg.static_scale], dtype=torch.float32, device=device)
        else:
            scale = torch.empty(cfg.tokens, 1, dtype=torch.float32, device=device)
        norm_out = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=device)
        sets.append((x, r, res_out, norm_out, scale))
    return sets, w


def sets_needed(cfg):
    per_set = cfg.tokens * cfg.hidden * 7
    return max(2, min(16, -(-4 * L2_BYTES // per_set)))


def time_calls(call, nsets, steps, warmup, barrier):
    """CUDA-event time of exactly `steps` calls after `warmup` calls; returns seconds."""
    for i in range(warmup):
        call(i % nsets)
    barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        call(i % nsets)
    end.record()
    torch.cuda.synchronize()
    barrier()
    return start.elapsed_time(end) * 1e-3


def max_over_ranks(seconds, world):
    if world == 1:
        return seconds
    import torch.distributed as dist
    t = torch.tensor([seconds], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_config(cfg, env, gpuk, rank, world, steps, warmup, barrier, graph=False, native=False):
    device = torch.device("cuda", torch.cuda.current_device())
    nsets = sets_needed(cfg)
    sets, w = make_sets(cfg, rank, world, nsets, device)
    fptr = env.fptr or 0

    def call(i):
        x, r, res_out, norm_out, scale = sets[i]
        gpuk.allreduce_rms(fptr, x, r, w, res_out, norm_out, scale, cfg.eps, cfg.quant_type)

    secs = max_over_ranks(time_calls(call, nsets, steps, warmup, barrier), world)
    out = {"workload": cfg.name, "us_per_call": secs / steps * 1e6, "buffer_sets": nsets}
    if graph:
        # the same calls replayed from a CUDA graph: launch overhead of the host wrapper removed
        g = torch.cuda.CUDAGraph()
        per_graph = nsets
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for i in range(per_graph):
                call(i)
            torch.cuda.synchronize()
            barrier()
            with torch.cuda.graph(g, stream=s):
                for i in range(per_graph):
                    call(i)
        torch.cuda.current_stream().wait_stream(s)
        reps = max(1, steps // per_graph)
        secs_g = max_over_ranks(time_calls(lambda i: g.replay(), 1, reps, max(3, warmup // per_graph), barrier), world)
        out["us_per_call_graph"] = secs_g / (reps * per_graph) * 1e6
    if world > 1 and native:
        # comparison on the same GPUs: NCCL all-reduce + the unfused PyTorch operator sequence
        x0, r0 = sets[0][0], sets[0][1]
        xn = x0.clone()

        def call_native(i):
            xn.copy_(x0)
            if cfg.quant_type == 4:
                import torch.distributed as dist
                dist.all_reduce(xn)
                ro = xn + r0
                v = ro.float().pow(2).mean(-1, keepdim=True)
                n = w * (ro * torch.rsqrt(v + cfg.eps)).to(ro.dtype)
                (n.float() / cfg.static_scale).clamp_(-448, 448).to(torch.float8_e4m3fn)
            else:
                env.allreduce_add_rms_native(xn, r0, w, cfg.eps, True)

        k = max(5, min(steps, 50))
        out["us_per_call_nccl_unfused"] = max_over_ranks(time_calls(call_native, 1, k, 3, barrier), world) / k * 1e6
    us = out.get("us_per_call_graph", out["us_per_call"]) if graph else out["us_per_call"]
    if world == 1:
        gbs = hbm_bytes(cfg.tokens, cfg.hidden) / (out["us_per_call"] * 1e-6) / 1e9
        peak, _ = measured_hbm_peak()
        out.update(hbm_gbs=gbs, frac_of_hbm_peak=gbs / peak)
    else:
        gbs = bus_bytes(cfg.tokens, cfg.hidden, world) / (us * 1e-6) / 1e9
        out.update(busbw_gbs=gbs, frac_of_nvlink_peak=gbs / NVLINK_PEER_COPY_GBS)
    del sets
    torch.cuda.empty_cache()
    return out


def run_e2e(cfg, env, rank, world, steps, warmup, barrier):
    """Public API with host buffers: the step's inputs start in pinned host memory and its three results end
    there (GPUKDistEnv.allreduce_add_rms_fused_host: rows pipelined in pieces over copy-in, kernel and copy-out
    streams); the timed region ends when the last result byte is on the host."""
    from gpuk_b200 import workloads as oin
    device = torch.device("cuda", torch.cuda.current_device())
    hx = oin.make_partial(cfg, rank, world).pin_memory()
    hr = oin.make_residual(cfg).pin_memory()
    w = oin.make_weight(cfg).to(device)
    o_res = torch.empty_like(hx).pin_memory()
    o_q = torch.empty(hx.shape, dtype=torch.float8_e4m3fn).pin_memory()
    o_s = torch.empty(cfg.tokens, 1, dtype=torch.float32).pin_memory()
    static = torch.tensor([cfg.static_scale], dtype=torch.float32, device=device) if cfg.quant_type == 4 else None
    chunks = int(os.environ.get("GPUK_E2E_CHUNKS", "4"))

    def call(_):
        env.allreduce_add_rms_fused_host(hx, hr, w, cfg.eps, (o_res, o_q, o_s), chunks=chunks, static_scale=static)

    secs = max_over_ranks(time_calls(call, 1, steps, warmup, barrier), world)
    h2d = hx.numel() * 2 + hr.numel() * 2
    d2h = o_res.numel() * 2 + o_q.numel() + (o_s.numel() * 4 if static is None else 0)
    return {"value": secs / steps * 1e6, "unit": "us/call", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "api": f"GPUKDistEnv.allreduce_add_rms_fused_host, {chunks} row pieces pipelined over three streams"}


def run_model(env, rank, world, steps, warmup, barrier):
    """Config 5: one decode step (batch 32, context 2048) of the 4-layer tensor-parallel decoder with the
    fused operator after attention and MLP of every layer, against the same model with NCCL all-reduce and
    unfused PyTorch operators; eager and replayed from a CUDA graph."""
    from gpuk_b200.tp_model import DecoderArgs, TPDecoder
    device = torch.device("cuda", torch.cuda.current_device())
    args = DecoderArgs()
    batch, ctx = 32, 2048
    out = {"workload": "c5_decoder_4layer_dim8192_ffn28672_b32_ctx2048", "batch": batch, "context": ctx, "fp8_activations": True}
    tokens = torch.randint(0, args.vocab_size, (batch, 1), generator=torch.Generator().manual_seed(11)).to(device)
    pos = torch.tensor([ctx], device=device)
    for name, fused in (("fused", True), ("nccl_unfused", False)):
        model = TPDecoder(args, env, device=device, fused=fused, fp8=True, max_batch=batch)
        model.fill_kv_cache(ctx)

        def step(_):
            model.forward(tokens, pos, cache_len=ctx + 1)

        secs = max_over_ranks(time_calls(step, 1, steps, warmup, barrier), world)
        out[f"us_per_step_{name}"] = secs / steps * 1e6
        try:
            g = torch.cuda.CUDAGraph()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                step(0)
                torch.cuda.synchronize()
                barrier()
                with torch.cuda.graph(g, stream=s):
                    step(0)
            torch.cuda.current_stream().wait_stream(s)
            secs = max_over_ranks(time_calls(lambda i: g.replay(), 1, steps, warmup, barrier), world)
            out[f"us_per_step_{name}_graph"] = secs / steps * 1e6
            del g
        except Exception as e:   # a capture failure is reported, not fatal
            out[f"graph_error_{name}"] = repr(e)[:200]
        del model
        torch.cuda.empty_cache()
        barrier()
    best = min(v for k, v in out.items() if k.startswith("us_per_step_fused"))
    out["tokens_per_s_fused"] = batch / (best * 1e-6)
    return out


# ---------------------------------------------------------------------------------------
# the reference's CPU path on the host cores
# ---------------------------------------------------------------------------------------
def _cpu_worker(rank, world, port, cfg_key, steps, warmup, threads, q):
    import torch.distributed as dist
    from oracle import epilogue_oracle as eo
    from gpuk_b200 import workloads as oin
    torch.set_num_threads(max(1, threads))
    cfg = oin.CONFIGS[cfg_key]
    if world > 1:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    x = oin.make_partial(cfg, rank, world)
    res = oin.make_residual(cfg)
    w = oin.make_weight(cfg)
    times = []
    for i in range(warmup + steps):
        xi = x.clone()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        if world > 1:
            dist.all_reduce(xi)                       # gpuk/__init__.py:156
        eo.add_rms_quant(xi, res, w, cfg.eps, cfg.quant_type, cfg.static_scale)   # :157-164
        if world > 1:
            dist.barrier()
        times.append(time.perf_counter() - t0)
    if rank == 0:
        q.put(times[warmup:])
    if world > 1:
        dist.destroy_process_group()


def cpu_reference_us(cfg_key, world, steps, warmup):
    """Median microseconds per call of the reference's CPU path: torch CPU operators, gloo
    all-reduce among `world` local processes sharing the host cores."""
    import socket
    import torch.multiprocessing as mp
    cores = os.cpu_count() or 1
    threads = max(1, cores // world)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env_backup = {k: os.environ.pop(k) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT",
                                                 "TORCHELASTIC_RUN_ID", "GROUP_RANK", "LOCAL_WORLD_SIZE")
                  if k in os.environ}
    try:
        procs = [ctx.Process(target=_cpu_worker, args=(r, world, port, cfg_key, steps, warmup, threads, q))
                 for r in range(world)]
        for p in procs:
            p.start()
        times = q.get(timeout=900)
        for p in procs:
            p.join(timeout=120)
    finally:
        os.environ.update(env_backup)
    return statistics.median(times) * 1e6, threads * world, threads


def reference_arm(args, rank, world):
    if rank != 0:
        return
    from gpuk_b200 import workloads as oin
    cfg = oin.CONFIGS[args.workload]
    steps = max(1, min(args.steps, 30))
    warmup = max(1, min(args.warmup, 5))
    us, cores, threads = cpu_reference_us(args.workload, world, steps, warmup)
    line = {
        "impl": "reference", "metric": "fused_ar_rmsnorm_fp8_us_per_call", "value": us, "unit": "us/call",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": us * 1e-3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg.name, "tokens": cfg.tokens, "hidden": cfg.hidden, "ranks": world,
                   "backend": "torch CPU operators" + (" + gloo all_reduce" if world > 1 else "")},
        "cpu_baseline": {"value": us, "unit": "us/call", "cores": cores, "kind": "port",
                         "sample": f"{steps} calls of the full {cfg.tokens}x{cfg.hidden} workload, "
                                   f"{world} process(es) x {threads} threads, median"},
        "e2e": {"value": us, "unit": "us/call", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_crossover(env, gpuk, rank, world, barrier, hidden=8192):
    """Microseconds per call (CUDA graph replay of the rotating buffer sets) of the three exchanges over
    the token counts between decode and prefill; used to place the thresholds between them."""
    from gpuk_b200 import workloads as oin
    rows = []
    have_sym = getattr(env, "_sym", None) is not None
    for tokens in (1, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192):
        cfg = oin.Config(9, f"x_{tokens}x{hidden}", tokens, hidden, 3)
        entry = {"tokens": tokens, "bytes": tokens * hidden * 2}
        for name, opts in (("one_shot", {"oneshot_max_bytes": 1 << 40, "sym_min_bytes": 0}),
                           ("two_shot", {"oneshot_max_bytes": 1, "sym_min_bytes": 0}),
                           ("symmetric", {"oneshot_max_bytes": 1, "sym_min_bytes": 1})):
            if name == "one_shot" and tokens * hidden * 2 > (2 << 20):
                continue
            if name == "symmetric" and not have_sym:
                continue
            for k, v in opts.items():
                env.set_option(k, v)
            steps = 400 if tokens <= 256 else (100 if tokens <= 2048 else 30)
            try:
                r = run_config(cfg, env, gpuk, rank, world, steps, 5, barrier, graph=True)
                entry[name] = r.get("us_per_call_graph", r["us_per_call"])
            except Exception as e:
                entry[name] = repr(e)[:120]
        rows.append(entry)
    env.set_option("oneshot_max_bytes", 0)
    env.set_option("sym_min_bytes", int(os.environ.get("GPUK_SYM_MIN_BYTES", "0")))
    return rows


# ---------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="gpuk_b200", choices=["gpuk_b200", "reference"])
    ap.add_argument("--workload", default="c3", choices=["c2", "c3", "c4", "c5"])
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-model", action="store_true", help="skip the decoder-model step (config 5) in the sweep")
    ap.add_argument("--crossover", action="store_true", help="also time one-shot / two-shot / symmetric over token counts")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, rank, max(world, args.gpus if world == 1 else world))
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")

    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("NCCL_DEBUG", "WARN")      # keeps NCCL's version banner off stdout
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        dist.init_process_group("gloo", rank=0, world_size=1)

    import gpuk_b200 as gpuk
    from gpuk_b200 import workloads as oin

    env = gpuk.GPUKDistEnv(group=None, device_id=local_rank)

    def barrier():
        if world > 1:
            dist.barrier()

    cfg = oin.CONFIGS[args.workload]
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    head = run_config(cfg, env, gpuk, rank, world, args.steps, args.warmup, barrier, native=True, graph=True)
    # keep the same kernel running a little longer so the 100 ms clock sampler sees it under load
    extra = max(0, int(0.4 / max(head["us_per_call"] * 1e-6, 1e-7)) - args.steps)
    if extra:
        run_config(cfg, env, gpuk, rank, world, min(extra, 200000), 3, barrier)
    clocks = sampler.stop() if rank == 0 else None

    e2e = run_e2e(cfg, env, rank, world, max(3, min(args.steps, 200)), 3, barrier)

    sweep = []
    if not args.no_sweep:
        for key in ("c2", "c3", "c4", "c5"):
            if key == args.workload:
                continue
            c = oin.CONFIGS[key]
            k = max(10, min(args.steps, 20000 if c.tokens <= 64 else (300 if c.tokens >= 8192 else 2000)))
            sweep.append(run_config(c, env, gpuk, rank, world, k, min(args.warmup, 20), barrier,
                                    graph=c.tokens <= 64, native=True))

        if not args.no_model:
            try:
                sweep.append(run_model(env, rank, world, max(10, min(args.steps, 100)), 5, barrier))
            except Exception as e:
                sweep.append({"workload": "c5_decoder", "error": repr(e)[:300]})

    crossover = run_crossover(env, gpuk, rank, world, barrier) if (args.crossover and world > 1) else None

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        us, cores, threads = cpu_reference_us(args.workload, 1, 12, 3)
        cpu = {"value": us, "unit": "us/call", "cores": cores, "kind": "port",
               "sample": f"12 calls of the full {cfg.tokens}x{cfg.hidden} workload (no exchange at one rank), median"}

    if rank == 0:
        us = head["us_per_call"]
        peak, peak_kind = measured_hbm_peak()
        if world == 1:
            ach = hbm_bytes(cfg.tokens, cfg.hidden) / (us * 1e-6) / 1e9
            roof = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                    "traffic": K1_DRAM_TRAFFIC_BYTES_PER_TOKEN_H8192 * cfg.tokens if cfg.hidden == 8192 else None,
                    "peak_kind": f"of {peak_kind}",
                    "algorithmic_bytes_per_launch": hbm_bytes(cfg.tokens, cfg.hidden),
                    "kernel": "fused_norm_quant_kernel"}
        else:
            ach = bus_bytes(cfg.tokens, cfg.hidden, world) / (us * 1e-6) / 1e9
            roof = {"bound": "nvlink", "achieved": ach, "peak": NVLINK_PEER_COPY_GBS, "unit": "GB/s",
                    "frac": ach / NVLINK_PEER_COPY_GBS, "traffic": None,
                    "peak_kind": "of measured peer copy per direction (nominal 900)",
                    "frac_of_sm_store_peak": ach / NVLINK_SM_STORE_GBS,
                    "algorithmic_bytes_per_launch": bus_bytes(cfg.tokens, cfg.hidden, world),
                    "kernel": "ar_kernel (two-shot, fused epilogue)"}
        line = {
            "metric": "fused_ar_rmsnorm_fp8_us_per_call", "value": us, "unit": "us/call", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": us * 1e-3, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": cfg.name, "tokens": cfg.tokens, "hidden": cfg.hidden, "ranks": world,
                       "quant": "per-token dynamic e4m3fn /448", "l2": f"rotating {head['buffer_sets']} buffer sets (> 4x L2)"},
            "busbw_gbs": roof["achieved"] if world > 1 else None,
            "roofline": roof, "clocks": clocks, "e2e": e2e, "gpu_launches": args.steps,
            "nccl_unfused_us_per_call": head.get("us_per_call_nccl_unfused"),
            "us_per_call_graph": head.get("us_per_call_graph"),
            "cpu_baseline": cpu, "sweep": sweep,
        }
        if crossover is not None:
            line["crossover"] = crossover
        print(json.dumps(line), flush=True)
    barrier()
    del env
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
