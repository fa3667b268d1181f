"""The caller of the fused operator: the tensor-parallel decoder of gpuk_b200/tp_model.py.

CPU (gloo, two ranks): sharding, KV cache and the reduce + add + norm hand-off are checked by
comparing a two-rank model with the one-rank model built from the same master weights.
GPU: the fused arrangement against the unfused one (NCCL all-reduce + PyTorch operators) on
the same weights, with and without FP8 activations.
"""
import os
import socket

import pytest
import torch

from gpuk_b200.tp_model import DecoderArgs, TPDecoder

SMALL = dict(dim=256, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=32, ffn_dim=512, vocab_size=128, max_seq_len=32)


class _Env:
    """What TPDecoder needs of a GPUKDistEnv when the fused operator is not used."""
    def __init__(self, rank, world):
        self.rank, self.world_size, self.group = rank, world, None


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _decode(model, tokens, prompt_len, steps):
    """Prefill `prompt_len` positions in one call, then `steps` single-token calls; returns all logits."""
    outs = [model.forward(tokens[:, :prompt_len], torch.arange(prompt_len, device=tokens.device))]
    for i in range(steps):
        p = prompt_len + i
        outs.append(model.forward(tokens[:, p:p + 1], torch.tensor([p], device=tokens.device), cache_len=p + 1))
    return torch.cat(outs, dim=1)


def _cpu_worker(rank, world, port, q):
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    args = DecoderArgs(dtype=torch.float32, **SMALL)
    model = TPDecoder(args, _Env(rank, world), device="cpu", fused=False, fp8=False, master_init=True, max_batch=3)
    tokens = torch.randint(0, args.vocab_size, (3, 12), generator=torch.Generator().manual_seed(5))
    logits = _decode(model, tokens, 8, 4)
    gathered = [torch.empty_like(logits) for _ in range(world)]
    dist.all_gather(gathered, logits)
    if rank == 0:
        q.put(torch.cat(gathered, dim=-1))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_one_rank_on_cpu():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_cpu_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    two = q.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
    assert all(p.exitcode == 0 for p in procs)
    args = DecoderArgs(dtype=torch.float32, **SMALL)
    one = TPDecoder(args, _Env(0, 1), device="cpu", fused=False, fp8=False, master_init=True, max_batch=3)
    tokens = torch.randint(0, args.vocab_size, (3, 12), generator=torch.Generator().manual_seed(5))
    want = _decode(one, tokens, 8, 4)
    assert two.shape == want.shape == (3, 12, args.vocab_size)
    torch.testing.assert_close(two, want, atol=2e-4, rtol=2e-4)


def test_decode_steps_match_a_single_prefill_on_cpu():
    """The KV cache path: prefill 8 + 4 decode steps = one 12-token call."""
    args = DecoderArgs(dtype=torch.float32, **SMALL)
    tokens = torch.randint(0, args.vocab_size, (2, 12), generator=torch.Generator().manual_seed(6))
    a = TPDecoder(args, _Env(0, 1), device="cpu", fused=False, fp8=False, master_init=True, max_batch=2)
    b = TPDecoder(args, _Env(0, 1), device="cpu", fused=False, fp8=False, master_init=True, max_batch=2)
    stepped = _decode(a, tokens, 8, 4)
    whole = b.forward(tokens, torch.arange(12))
    torch.testing.assert_close(stepped, whole, atol=2e-4, rtol=2e-4)


# ------------------------------------------------------------------------------------------
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0
MID = dict(dim=2048, n_layers=2, n_heads=16, n_kv_heads=4, head_dim=128, ffn_dim=4096, vocab_size=1024, max_seq_len=160)


def _gpu_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    import gpuk_b200
    env = _RecordingEnv(gpuk_b200.GPUKDistEnv(group=None, device_id=rank, max_size_in_bytes=16 << 20))
    failures = []

    def gather(p):
        parts = [torch.empty_like(p) for _ in range(world)]
        dist.all_gather(parts, p)
        return parts

    try:
        args = DecoderArgs(**MID)
        tokens = torch.randint(0, args.vocab_size, (4, 1), generator=torch.Generator().manual_seed(3)).cuda()
        for fp8 in (False, True):
            logits = []
            for fused in (True, False):
                env.calls.clear()
                m = TPDecoder(args, env, device=f"cuda:{rank}", fused=fused, fp8=fp8, max_batch=4)
                m.fill_kv_cache(128)
                pos = torch.tensor([128], device=f"cuda:{rank}")
                logits.append(m.forward(tokens, pos, cache_len=129).float())
                if fused:
                    torch.cuda.synchronize()
                    try:
                        _check_hand_offs(env.calls, gather)
                    except AssertionError as e:   # pragma: no cover
                        failures.append(f"fp8={fp8}: hand-off parity: {e}")
            torch.cuda.synchronize()
            err = (logits[0] - logits[1]).abs().max().item()
            ref = logits[1].abs().max().item()
            # two-rank bf16 sums are a single add, so the arrangements differ only by FP8 rounding of ties
            if not err <= (0.08 if fp8 else 0.03) * max(ref, 1e-3):
                failures.append(f"fp8={fp8}: fused vs unfused logits differ by {err} (scale {ref})")
    except Exception as e:   # pragma: no cover
        failures.append(repr(e))
    finally:
        q.put((rank, failures))
        env.barrier()
        del env
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.skipif(NGPU < 2, reason="needs at least two GPUs")
def test_fused_decoder_matches_unfused_on_two_gpus():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gpu_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
    for rank, failures in results:
        assert not failures, (rank, failures)


class _RecordingEnv:
    """Wraps a GPUKDistEnv and keeps inputs and results of every fused hand-off the decoder makes."""

    def __init__(self, env):
        self._env = env
        self.calls = []

    def __getattr__(self, name):
        return getattr(self._env, name)

    def allreduce_add_rms_fused(self, partial, h, weight, eps, fp8_out=False, **kw):
        p, r = partial.clone(), h.clone()
        out = self._env.allreduce_add_rms_fused(partial, h, weight, eps, fp8_out, **kw)
        self.calls.append((p, r, weight, eps, fp8_out, tuple(t.clone() for t in out)))
        return out


def _check_hand_offs(calls, gather):
    """Every recorded hand-off against the oracle with the parity bars of the operator itself (so a wrong
    scale on a single row of a single layer fails, which a tolerance on the logits would not notice)."""
    from oracle import epilogue_oracle as eo
    from tests import util
    assert calls
    for p, r, weight, eps, fp8_out, out in calls:
        parts = [t.cpu() for t in gather(p)]
        quant = 3 if fp8_out else 0
        want = eo.epilogue_t1(parts, r.cpu(), weight.cpu(), eps, quant)
        got = (out[0].cpu(), out[1].cpu(), out[2].cpu() if fp8_out else None)
        util.check_against_oracle(got, want, quant)


@pytest.mark.gpu
def test_every_fused_hand_off_of_the_decoder_meets_the_operator_parity_bars_on_one_gpu():
    import torch.distributed as dist
    import gpuk_b200
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(_free_port()))
        dist.init_process_group("gloo", rank=0, world_size=1)
    env = _RecordingEnv(gpuk_b200.GPUKDistEnv(group=None, device_id=0))
    args = DecoderArgs(**MID)
    tokens = torch.randint(0, args.vocab_size, (4, 1), generator=torch.Generator().manual_seed(3)).cuda()
    for fp8 in (False, True):
        env.calls.clear()
        m = TPDecoder(args, env, device="cuda:0", fused=True, fp8=fp8, max_batch=4)
        m.fill_kv_cache(128)
        m.forward(tokens, torch.tensor([128], device="cuda:0"), cache_len=129)
        torch.cuda.synchronize()
        assert len(env.calls) >= 2 * args.n_layers
        _check_hand_offs(env.calls, lambda p: [p])


@pytest.mark.gpu
def test_fused_decoder_on_one_gpu():
    """A group of one: the no-communication kernel carries both hand-offs of every layer."""
    import torch.distributed as dist
    import gpuk_b200
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(_free_port()))
        dist.init_process_group("gloo", rank=0, world_size=1)
    env = gpuk_b200.GPUKDistEnv(group=None, device_id=0)
    args = DecoderArgs(**MID)
    tokens = torch.randint(0, args.vocab_size, (4, 1), generator=torch.Generator().manual_seed(3)).cuda()
    for fp8 in (False, True):
        logits = []
        for fused in (True, False):
            m = TPDecoder(args, env, device="cuda:0", fused=fused, fp8=fp8, max_batch=4)
            m.fill_kv_cache(128)
            logits.append(m.forward(tokens, torch.tensor([128], device="cuda:0"), cache_len=129).float())
        err = (logits[0] - logits[1]).abs().max().item()
        ref = logits[1].abs().max().item()
        assert err <= (0.08 if fp8 else 0.03) * max(ref, 1e-3), (fp8, err, ref)


@pytest.mark.gpu
def test_decoder_with_this_librarys_fp8_linear_matches_the_library_gemm_on_one_gpu():
    """own_fp8_gemm=True routes q|k|v, w1|w3 and the vocabulary projection of a decode step through
    gpuk_fp8_linear_skinny (blocked weights); both GEMMs round fp32-accurate sums once, so the logits agree closely."""
    import torch.distributed as dist
    import gpuk_b200
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(_free_port()))
        dist.init_process_group("gloo", rank=0, world_size=1)
    env = gpuk_b200.GPUKDistEnv(group=None, device_id=0)
    args = DecoderArgs(**MID)
    tokens = torch.randint(0, args.vocab_size, (4, 1), generator=torch.Generator().manual_seed(3)).cuda()
    logits = []
    for own in (True, False):
        m = TPDecoder(args, env, device="cuda:0", fused=True, fp8=True, max_batch=4, own_fp8_gemm=own)
        m.fill_kv_cache(128)
        logits.append(m.forward(tokens, torch.tensor([128], device="cuda:0"), cache_len=129).float())
        if own:
            assert m.layers[0]["wqkv"].w_packed is not None      # the kernel was taken, not the library fallback
    # a GEMM output one bf16 step away can move an FP8 code of the next hand-off: the largest deviation is what one
    # such flip does to a logit, the typical one far smaller
    diff = (logits[0] - logits[1]).abs()
    ref = logits[1].abs().max().item()
    assert diff.max().item() <= 0.06 * max(ref, 1e-3), (diff.max().item(), ref)
    assert diff.mean().item() <= 0.01 * max(ref, 1e-3), (diff.mean().item(), ref)
