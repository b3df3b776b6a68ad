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
