"""DDP communication hook: on CPU ranks (gloo + host-rank ring) and on GPUs."""
import pytest
import torch

from mp_util import run_ranks


def _train(rank, world, device_type):
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    from tirocinio_triennale_b200.models import GPT2, GPT2Config
    from tirocinio_triennale_b200.parallel import CompressedHookState, compressed_allreduce_hook

    device = torch.device(device_type, rank) if device_type == "cuda" else torch.device("cpu")
    eb = 1e-6

    def make(hook):
        torch.manual_seed(0)
        m = GPT2(GPT2Config.tiny()).to(device)
        d = DDP(m, device_ids=[rank] if device_type == "cuda" else None, bucket_cap_mb=0.05)
        st = None
        if hook:
            st = CompressedHookState(eb=eb, max_bucket_elems=1 << 20, min_compress_elems=1)
            d.register_comm_hook(st, compressed_allreduce_hook)
        return m, d, st

    m1, d1, st = make(True)
    m2, d2, _ = make(False)
    g = torch.Generator().manual_seed(10 + rank)
    for _ in range(3):
        tok = torch.randint(0, 257, (4, 33), generator=g).to(device)
        for d in (d1, d2):
            d.zero_grad(set_to_none=True)
            d(tok[:, :-1], tok[:, 1:]).backward()
        if device_type == "cuda":
            torch.cuda.synchronize()
        for p1, p2 in zip(m1.parameters(), m2.parameters()):
            # averaged gradients agree within the error bound (world quantisation errors / world)
            assert (p1.grad - p2.grad).abs().max().item() <= eb * 1.01 + 1e-7
    assert st.compressed_calls > 0
    # every rank holds the same averaged gradient bit for bit
    flat = torch.cat([p.grad.reshape(-1) for p in m1.parameters()]).cpu()
    gathered = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat) if device_type == "cpu" else dist.all_gather(
        [t.to(device) for t in gathered], flat.to(device))
    if device_type == "cpu":
        for t in gathered:
            assert torch.equal(t, flat)
    st.close()


def test_hook_on_cpu_ranks():
    run_ranks(_train, 2, args=("cpu",))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_hook_on_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_train, 2, args=("cuda",), backend="nccl")


def _overlap(rank, world):
    """The hook must not order the backward stream behind the collective it launches."""
    from tirocinio_triennale_b200.parallel import CompressedHookState
    from tirocinio_triennale_b200.parallel.ddp_hook import launch_bucket

    n = 16 * 1024 * 1024
    state = CompressedHookState(eb=1e-4, max_bucket_elems=n)
    buf = torch.randn(n, device="cuda") * 0.01
    launch_bucket(state, buf, 1).wait()
    torch.cuda.synchronize()
    cur = torch.cuda.current_stream()
    ev_mid, ev_end, ev_after = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    torch.cuda._sleep(4_000_000)  # ~2 ms on the backward stream: the collective is queued behind it
    fut = launch_bucket(state, buf, 1)
    ev_mid.record(cur)  # what backward queues next
    torch.cuda._sleep(400_000)
    with torch.cuda.stream(state.stream):
        ev_end.record()  # end of the collective
    fut.wait()  # the consumer of the bucket is ordered behind it, without blocking the host
    ev_after.record(cur)
    torch.cuda.synchronize()
    # the backward stream went on while the collective (tens of microseconds for 64 MiB) was running
    assert ev_mid.elapsed_time(ev_end) > 0.02, ev_mid.elapsed_time(ev_end)
    assert ev_end.elapsed_time(ev_after) >= 0.0
    state.check()
    state.close()


@pytest.mark.gpu
def test_hook_does_not_block_the_backward_stream():
    run_ranks(_overlap, 1, backend="nccl")


def _busy_sms(rank, world):
    """Collective launched while another stream keeps every SM busy with GEMMs: the CTAs get their SM
    slots late, nothing may time out and the result is the one of an idle GPU."""
    from tirocinio_triennale_b200.parallel import CompressedAllreduce

    n = 4 * 1024 * 1024
    ar = CompressedAllreduce(n, timeout_ms=2000)
    x = torch.randn(n, device="cuda") * 0.01
    want = ar.allreduce(x, torch.empty_like(x), 1e-4).clone()
    a = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    got = torch.empty_like(x)
    with torch.cuda.stream(side):
        for _ in range(12):
            a @ a
    for _ in range(6):
        ar.allreduce(x, got, 1e-4)
    torch.cuda.synchronize()
    assert ar.status() == 0
    assert torch.equal(got, want)
    ar.close()


@pytest.mark.gpu
def test_collective_beside_a_gemm_stream():
    run_ranks(_busy_sms, 1, backend="nccl")
