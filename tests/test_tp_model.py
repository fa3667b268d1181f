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
    env = gpuk_b200.GPUKDistEnv(group=None, device_id=rank, max_size_in_bytes=16 << 20)
    failures = []
    try:
        args = DecoderArgs(**MID)
        tokens = torch.randint(0, args.vocab_size, (4, 1), generator=torch.Generator().manual_seed(3)).cuda()
        for fp8 in (False, True):
            logits = []
            for fused in (True, False):
                m = TPDecoder(args, env, device=f"cuda:{rank}", fused=fused, fp8=fp8, max_batch=4)
                m.fill_kv_cache(128)
                pos = torch.tensor([128], device=f"cuda:{rank}")
                logits.append(m.forward(tokens, pos, cache_len=129).float())
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
