"""Host-side rules of Buffer / ElasticBuffer with a stub transport (CPU, single process).

The stub records calls and returns CPU tensors of the right shapes; it validates nothing about
data movement (the Gloo and GPU tests do that).  What is pinned down here is the contract the
reference documents in docs/api.md and checks with mocks in tests/unit/test_deepep.py: roles,
one pending exchange, receipt identity, capture restrictions, argument validation, collective
preflight.
"""

import pytest
import torch

import afdep_b200.buffer as buffer_mod
from afdep_b200 import Buffer, Config, ElasticBuffer
from afdep_b200.parallel.control import LocalControl


class StubTransport:
    def __init__(self, *, control, group, config, num_sms, options):
        self.config, self.rank = config, control.rank
        self.topk_idx_dtype, self.float32, self.bfloat16 = torch.int64, torch.float32, torch.bfloat16
        self.payload_dtype = torch.float8_e4m3fn if config.is_fp8 else torch.bfloat16
        self.num_buffer_bytes, self.comm_stream, self.device = 4096, None, None
        self.capturing, self.calls, self.closed = False, [], False

    def check_device(self): ...
    def raise_status(self): ...
    def is_capturing(self): return self.capturing
    def on_device(self, t): return True
    def stats(self): return {"launches": len(self.calls)}

    def empty_source(self):
        c = self.config
        return (torch.empty((0, c.hidden_size), dtype=self.payload_dtype), torch.empty((0, c.scale_groups)) if c.is_fp8 else None,
                torch.empty((0, c.top_k), dtype=torch.int64), torch.empty((0, c.top_k)))

    def empty_receive(self):
        c = self.config
        return (torch.empty((0, c.hidden_size), dtype=self.payload_dtype), torch.empty((0, c.scale_groups)) if c.is_fp8 else None,
                torch.empty((0,)), torch.zeros((c.experts_per_rank,), dtype=torch.int32), torch.empty((0, 2), dtype=torch.int32))

    def empty_output(self):
        return torch.empty((0, self.config.hidden_size), dtype=torch.bfloat16)

    def source_dispatch(self, x, x_scale, ids, w, *, bucket):
        self.calls.append(("dispatch", x.shape[0], bucket, x_scale))

    def worker_receive(self, *, bucket, read_host_counts):
        c = self.config
        rows = c.receive_rows(bucket)
        self.calls.append(("receive", bucket, read_host_counts))
        return (torch.zeros((rows, c.hidden_size), dtype=self.payload_dtype), torch.zeros((rows, c.scale_groups)) if c.is_fp8 else None,
                torch.zeros((rows,)), torch.zeros((c.experts_per_rank,), dtype=torch.int32),
                [0] * c.experts_per_rank if read_host_counts else [], torch.zeros((rows, 2), dtype=torch.int32))

    def worker_reply(self, rows): self.calls.append(("reply", tuple(rows.shape)))
    def source_collect(self, n):
        self.calls.append(("collect", n))
        return torch.zeros((n, self.config.hidden_size), dtype=torch.bfloat16)
    def close(self): self.closed = True


@pytest.fixture
def stub(monkeypatch):
    monkeypatch.setattr(buffer_mod, "_make_transport", lambda kind, **kw: StubTransport(**kw))
    monkeypatch.setattr(LocalControl, "check_backend", lambda self, backend: None)
    monkeypatch.setattr(LocalControl, "local_probe", lambda self, backend: {"sms": 148, "device": None, "source": "x"})


def make(rank, **kw):
    cfg = Config(**({"capacity_tokens_per_rank": 16, "hidden_size": 256, "num_experts": 16, "top_k": 4, "ffn_ranks": 2, "attention_ranks": 2} | kw))
    return Buffer(group=None, config=cfg, backend="stub", _control=LocalControl(rank, cfg.world_size)), cfg


def tokens(cfg, n, dtype=torch.bfloat16):
    return torch.zeros((n, cfg.hidden_size), dtype=dtype), torch.zeros((n, cfg.top_k), dtype=torch.int64), torch.zeros((n, cfg.top_k))


def test_roles_follow_rank_order_and_defaults(stub):
    ffn, cfg = make(1)
    att, _ = make(2)
    assert (ffn.role, ffn.role_rank, att.role, att.role_rank) == ("ffn", 1, "attention", 0)
    assert att.transport._num_sms() == 27          # 24/132 of a 148-SM device
    assert att.physical_domain == (1, 4) and att.num_buffer_bytes == 4096
    with pytest.raises(RuntimeError, match="requires the ffn role"):
        att.worker_receive(bucket=8)
    with pytest.raises(RuntimeError, match="requires the attention role"):
        ffn.source_dispatch(*tokens(cfg, 2), bucket=8)


def test_source_owns_no_receive_rows_and_collects_in_token_order(stub):
    att, cfg = make(3)
    att.source_dispatch(*tokens(cfg, 5), bucket=8, read_host_counts=True)
    pending = att.transport._pending
    assert pending.recv_shape == (0, 256) and pending.num_tokens == 5
    out = att.source_collect()
    assert out.shape == (5, 256) and att.transport._pending is None
    with pytest.raises(RuntimeError, match="matching dispatch"):
        att.source_collect()


def test_one_pending_exchange_and_receipt_identity(stub):
    ffn, cfg = make(0)
    rec = ffn.worker_receive(bucket=8)
    assert rec.recv_x.shape[0] == cfg.receive_rows(8) and rec.receipt is rec.handle
    with pytest.raises(RuntimeError, match="previous exchange"):
        ffn.worker_receive(bucket=8)
    other, _ = make(1)
    foreign = other.worker_receive(bucket=8)
    rows = torch.zeros(rec.receipt.recv_shape, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="Handle does not belong"):
        ffn.worker_reply(rows, foreign.receipt)
    with pytest.raises(ValueError, match="dtype, shape"):
        ffn.worker_reply(rows[:-1], rec.receipt)
    ffn.worker_reply(rows, rec.receipt)
    with pytest.raises(ValueError, match="Handle does not belong"):
        ffn.worker_reply(rows, rec.receipt)        # already consumed


def test_low_level_facade_rejects_tokens_on_ffn_ranks(stub):
    cfg = Config(16, 256, 16, 4, 2, 2)
    eb = ElasticBuffer(group=None, capacity_tokens_per_rank=16, hidden_size=256, num_experts=cfg.logical_experts, top_k=4,
                       allow_hybrid_mode=True, rdma_traffic_class=0, cpu_timeout_s=5, gpu_timeout_s=5, role_aware=True, ffn_ranks=2,
                       backend="stub", _control=LocalControl(0, 4))
    x, ids, w = tokens(cfg, 2)
    with pytest.raises(ValueError, match="cannot originate tokens"):
        eb.dispatch(x, None, ids, w, bucket=8, expert_alignment=128, do_cpu_sync=False)
    with pytest.raises(ValueError, match="bucket must be positive"):
        eb.dispatch(x[:0], None, ids[:0], w[:0], bucket=17, expert_alignment=128, do_cpu_sync=False)
    with pytest.raises(ValueError, match="expert_alignment differs"):
        eb.dispatch(x[:0], None, ids[:0], w[:0], bucket=8, expert_alignment=64, do_cpu_sync=False)
    with pytest.raises(ValueError, match="do_cpu_sync must be a boolean"):
        eb.dispatch(x[:0], None, ids[:0], w[:0], bucket=8, expert_alignment=128, do_cpu_sync=1)
    eb.close()
    eb.destroy()            # alias, idempotent
    with pytest.raises(RuntimeError, match="closed"):
        eb.dispatch(x[:0], None, ids[:0], w[:0], bucket=8, expert_alignment=128, do_cpu_sync=False)


def test_capture_forbids_host_counts_and_close(stub):
    ffn, _ = make(0)
    ffn._t.capturing = True
    with pytest.raises(RuntimeError, match="unavailable during CUDA capture"):
        ffn.worker_receive(bucket=8, read_host_counts=True)
    rec = ffn.worker_receive(bucket=8)
    with pytest.raises(RuntimeError, match="outside CUDA graph capture"):
        ffn.close()
    ffn._t.capturing = False
    with pytest.raises(RuntimeError, match="pending exchange"):
        ffn.close()
    ffn.worker_reply(torch.zeros(rec.receipt.recv_shape, dtype=torch.bfloat16), rec.receipt)
    ffn.close()
    assert ffn._t.closed
    ffn.close()


def test_payload_validation(stub):
    att, cfg = make(2)
    x, ids, w = tokens(cfg, 4)
    with pytest.raises(ValueError, match="exceeds its bucket"):
        att.source_dispatch(x, ids, w, bucket=2)
    with pytest.raises(ValueError, match="dtype, shape"):
        att.source_dispatch(x.float(), ids, w, bucket=8)
    with pytest.raises(ValueError, match="dtype, shape"):
        att.source_dispatch(x, ids.int(), w, bucket=8)
    with pytest.raises(ValueError, match="dtype, shape"):
        att.source_dispatch(x.t().contiguous().t(), ids, w, bucket=8)          # not contiguous
    with pytest.raises(ValueError, match="FP32 block128 scales"):
        att.source_dispatch(x, ids, w, torch.zeros((4, 2)), bucket=8)          # scales on a BF16 buffer
    with pytest.raises(ValueError, match="shape \\[tokens,hidden\\]"):
        att.source_dispatch(x[0], ids, w, bucket=8)
    fp8, cfg8 = make(2, payload="fp8")
    x8 = torch.zeros((4, 256), dtype=torch.float8_e4m3fn)
    with pytest.raises(ValueError, match="FP32 block128 scales"):
        fp8.source_dispatch(x8, ids, w, bucket=8)
    strided = torch.zeros((4, 4))[:, ::2]                                       # strided scale views are legal
    fp8.source_dispatch(x8, ids, w, strided, bucket=8)
    assert fp8._t.calls[-1][3] is strided                                       # passed through, not copied


def test_preflight_errors_are_collected_for_every_rank(stub):
    common = dict(group=None, capacity_tokens_per_rank=16, hidden_size=256, top_k=16, allow_hybrid_mode=True,
                  rdma_traffic_class=0, cpu_timeout_s=5, gpu_timeout_s=5, backend="stub", _control=LocalControl(2, 4))
    with pytest.raises(RuntimeError, match="explicit ffn_ranks"):
        ElasticBuffer(num_experts=32, role_aware=True, **common)
    with pytest.raises(RuntimeError, match="rank 0: .*rank 3: "):               # every rank reports
        ElasticBuffer(num_experts=32, role_aware=True, **common)
    with pytest.raises(RuntimeError, match="exceeds the real FFN expert count"):
        ElasticBuffer(num_experts=16, role_aware=True, ffn_ranks=2, **common)
    with pytest.raises(RuntimeError, match="divide evenly over the group"):
        ElasticBuffer(num_experts=30, role_aware=True, ffn_ranks=2, **(common | {"top_k": 2}))
    with pytest.raises(RuntimeError, match="at least two ranks"):
        ElasticBuffer(num_experts=8, role_aware=True, ffn_ranks=1, **(common | {"top_k": 2, "_control": LocalControl(0, 1)}))
