"""Four CPU ranks over Gloo: the role API end to end on the pure-torch transport.

Covers the first benchmark configuration (2 FFN + 2 attention ranks, hidden 128*, 8 experts,
top-2, 16 tokens, bucket 16; *hidden is 256 here because the API requires multiples of 256)
with the closed form ``out == sum_k w_k * (e_k + 1) * x``, plus the host-side rules of the
Buffer that the reference checks with mocks: single pending exchange, receipt identity,
collective close.
"""

import pytest
import torch

from afdep_b200 import Buffer, Config
from afdep_b200.utils import oracle, synthetic
from tests._dist import run_ranks


def _exchange(rank, world, payload, read_host_counts):
    import torch.distributed as dist

    packed = payload == "fp8-packed"          # FP8 rows whose scales travel as packed exponent bytes
    cfg = Config(16, 256, 8, 2, 2, 2, expert_alignment=4, payload="fp8" if packed else payload,
                 scale_format="ue8m0x4" if packed else "fp32")
    buf = Buffer(group=dist.group.WORLD, config=cfg, backend="gloo")
    assert buf.role == ("ffn" if rank < 2 else "attention")
    for epoch in range(3):
        batches = [synthetic.exact_batch(cfg, 16, a, epoch, active=16 - 5 * a * (epoch % 2)) for a in range(2)]
        if buf.role == "attention":
            x, ids, w, scale = batches[buf.role_rank]
            if packed:
                assert scale.dtype == torch.int32 and scale.shape == (x.shape[0], 1)
                with pytest.raises(ValueError, match="dtype, shape"):
                    buf.source_dispatch(x, ids, w, oracle.dequantize(torch.ones_like(x), scale)[:, :2].contiguous(), bucket=16)
            buf.source_dispatch(x, ids, w, scale, bucket=16, read_host_counts=read_host_counts)
            with pytest.raises(RuntimeError, match="previous exchange"):
                buf.source_dispatch(x, ids, w, scale, bucket=16)
            out = buf.source_collect()
            factor = torch.where(ids >= 0, (ids + 1).float() * w, torch.zeros_like(w)).sum(dim=1)
            expect = (oracle.dequantize(x, scale) * factor[:, None]).to(torch.bfloat16)
            torch.testing.assert_close(out, expect, rtol=0, atol=0)
            torch.testing.assert_close(out, oracle.expected_combine(cfg, oracle.SourceBatch(x, ids, w, scale)), rtol=0, atol=0)
        else:
            rec = buf.worker_receive(bucket=16, read_host_counts=read_host_counts)
            exp = oracle.expected_receive(cfg, buf.role_rank, [oracle.SourceBatch(*b[:3], b[3]) for b in batches], rows=rec.recv_x.shape[0])
            assert torch.equal(rec.recv_count_psum.long(), exp.layout.ends)
            v = exp.valid
            assert torch.equal(rec.recv_x[v].float(), exp.recv_x[v].float())
            if cfg.is_fp8:
                assert rec.recv_scale.dtype == (torch.int32 if packed else torch.float32)
                assert torch.equal(rec.recv_scale[v], exp.recv_scale[v])
            assert torch.equal(rec.recv_topk_weights[v], exp.recv_weights[v])
            assert torch.equal(rec.handle.recv_src_metadata[v], exp.recv_src[v])
            if read_host_counts:
                assert rec.recv_counts_host == exp.layout.aligned_counts
                assert rec.recv_x.shape[0] == exp.layout.rows_exact
            else:
                assert rec.recv_x.shape[0] == cfg.receive_rows(16)
            rows = oracle.synthetic_expert_rows(cfg, buf.role_rank, rec.recv_x, rec.recv_scale, rec.recv_topk_weights, rec.recv_count_psum)
            with pytest.raises(ValueError, match="Handle does not belong"):
                buf.worker_reply(rows, type(rec.receipt)(**{**rec.receipt.__dict__, "_owner": object()}))
            buf.worker_reply(rows, rec.receipt)
    buf.close()
    buf.close()   # idempotent


@pytest.mark.parametrize("payload", ["bf16", "fp8", "fp8-packed"])
@pytest.mark.parametrize("read_host_counts", [False, True])
def test_four_rank_exchange(payload, read_host_counts):
    run_ranks(_exchange, 4, payload, read_host_counts)


def _mismatch(rank, world):
    import torch.distributed as dist

    cfg = Config(16, 256, 8, 2, 2, 2, expert_alignment=4 if rank else 8)
    with pytest.raises(ValueError, match="same Config"):
        Buffer(group=dist.group.WORLD, config=cfg, backend="gloo")


def test_configs_must_agree():
    run_ranks(_mismatch, 4)


def _pending_close(rank, world):
    import torch.distributed as dist

    cfg = Config(8, 256, 8, 2, 2, 2, expert_alignment=1)
    buf = Buffer(group=dist.group.WORLD, config=cfg, backend="gloo")
    batch = synthetic.exact_batch(cfg, 8, 0, 0)
    if buf.role == "attention":
        buf.source_dispatch(*batch[:3], bucket=8)
        with pytest.raises(RuntimeError, match="requires the ffn role"):
            buf.worker_receive(bucket=8)
    rec = buf.worker_receive(bucket=8) if buf.role == "ffn" else None
    with pytest.raises(RuntimeError, match="pending exchange"):
        buf.close()
    if rec is not None:
        buf.worker_reply(torch.zeros(rec.receipt.recv_shape, dtype=torch.bfloat16), rec.receipt)
    else:
        buf.source_collect()
    buf.close()


def test_close_refuses_pending_exchange_on_every_rank():
    run_ranks(_pending_close, 4)


def _withheld_reply(rank, world):
    """Failure made on the host: FFN rank 0 receives and then never replies.  The attention
    ranks are waiting for its rows; their next collective call must fail within the group's
    timeout instead of blocking for good, and every process must still be able to leave."""
    import datetime

    import torch.distributed as dist

    group = dist.new_group(list(range(world)), backend="gloo", timeout=datetime.timedelta(seconds=4))
    cfg = Config(8, 256, 8, 2, 2, 2, expert_alignment=1)
    buf = Buffer(group=group, config=cfg, backend="gloo")
    batch = synthetic.exact_batch(cfg, 8, 0, 0)
    if buf.role == "attention":
        buf.source_dispatch(*batch[:3], bucket=8)
        with pytest.raises(RuntimeError):
            buf.source_collect()           # rows of FFN rank 0 never come
    else:
        rec = buf.worker_receive(bucket=8)
        if buf.role_rank == 1:
            rows = oracle.synthetic_expert_rows(cfg, 1, rec.recv_x, rec.recv_scale, rec.recv_topk_weights, rec.recv_count_psum)
            try:
                buf.worker_reply(rows, rec.receipt)
            except RuntimeError:
                pass      # its receivers were stuck behind the failed rank: a bounded failure too, not a hang
        # role rank 0 "fails" here: it keeps its receipt and says nothing
    # the Buffer is not closed (its exchange cannot complete); the job's own group is still healthy


def test_withheld_reply_fails_within_the_group_timeout():
    run_ranks(_withheld_reply, 4, timeout=120)
