"""Stream files (compressed tensors on disk) and checkpoint / resume of the data-parallel harness."""
import argparse

import numpy as np
import pytest
import torch

from mp_util import run_ranks
from tirocinio_triennale_b200 import ops
from tirocinio_triennale_b200.ops import stream_io


def test_tensor_file_roundtrip(tmp_path):
    g = torch.Generator().manual_seed(3)
    t = torch.randn(37, 129, generator=g) * 0.05
    eb = 1e-3
    nbytes = stream_io.save_tensor(tmp_path / "t.hcz", t, eb)
    assert nbytes < t.numel() * 4  # it did compress
    back = stream_io.load_tensor(tmp_path / "t.hcz")
    assert back.shape == t.shape and back.dtype == torch.float32
    assert (back - t).abs().max().item() <= eb * 1.0001
    # the body is the codec's stream, byte for byte
    raw = (tmp_path / "t.hcz").read_bytes()
    n, sbytes, eb_f, mode, shape = stream_io.unpack_header(raw)
    assert (n, mode, shape) == (t.numel(), "outlier", (37, 129)) and abs(eb_f - eb) < 1e-9
    want = ops.cpu_compress(t.reshape(-1).numpy(), eb)
    assert sbytes == want.size
    np.testing.assert_array_equal(np.frombuffer(raw, dtype=np.uint8, offset=stream_io.HEADER.size), want)


def test_bad_files_are_rejected(tmp_path):
    t = torch.linspace(-1, 1, 5000)
    raw = stream_io.dumps_tensor(t, 1e-3)
    with pytest.raises(ValueError):
        stream_io.loads_tensor(b"NOTASTRM" + raw[8:])
    with pytest.raises(ValueError):
        stream_io.loads_tensor(raw[: len(raw) // 2])


def test_state_dict_roundtrip(tmp_path):
    g = torch.Generator().manual_seed(5)
    state = {"w": torch.randn(64, 128, generator=g) * 0.02, "b": torch.randn(16, generator=g),
             "steps": torch.tensor(7), "ids": torch.arange(10000), "name": "x"}
    stats = stream_io.save_state(tmp_path / "s.zip", state, eb=1e-4)
    assert stats["raw_bytes"] == 64 * 128 * 4 and 0 < stats["file_bytes"] < stats["raw_bytes"]
    back = stream_io.load_state(tmp_path / "s.zip")
    assert set(back) == set(state) and back["name"] == "x"
    assert (back["w"] - state["w"]).abs().max().item() <= 1e-4 * 1.0001
    for k in ("b", "steps", "ids"):  # small or non-float tensors are stored verbatim
        assert torch.equal(back[k], state[k])


def _resume_worker(rank, world, prefix):
    from tirocinio_triennale_b200.models import train_dp

    def args(**kw):
        base = dict(model="tiny", steps=4, warmup=0, batch=2, seq=32, eb=1e-6, lr=1e-3, bucket_mb=0.05, cpu=True,
                    save=None, resume=None, save_compressed_eb=0.0)
        base.update(kw)
        return argparse.Namespace(**base)

    dev = torch.device("cpu")
    for compressed in (True, False):
        whole = train_dp.run(args(steps=4), compressed, rank, world, dev)
        first = train_dp.run(args(steps=2, save=prefix, save_compressed_eb=1e-5), compressed, rank, world, dev)
        rest = train_dp.run(args(steps=2, resume=prefix), compressed, rank, world, dev)
        assert first["steps_done"] == 2 and rest["steps_done"] == 4
        # the interrupted run continues exactly where the uninterrupted one went
        assert rest["last_loss_rank0"] == whole["last_loss_rank0"]
        if rank == 0:
            ck = first["compressed_checkpoint"]
            assert 0 < ck["file_bytes"] < ck["raw_bytes"]


def test_resume_continues_bit_for_bit(tmp_path):
    run_ranks(_resume_worker, 2, args=(str(tmp_path / "ck"),))
