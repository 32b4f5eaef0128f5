"""CPU unit tests of ``CudaBuffer`` wiring with test doubles (no GPU, no extension).

Mirrors the reference's unit tier (tests/unit/test_cuda_bootstrap.py, test_cuda_dispatch.py,
test_cuda_combine.py): two threads act as two ranks over a condition-variable rendezvous, the native
window and the CUDA runtime are fakes that record what happened.
"""

import pickle
import threading
from types import SimpleNamespace

import pytest
import torch

from nanoep_b200 import EPConfig
from nanoep_b200.parallel import bootstrap, cuda_buffer
from nanoep_b200.parallel.cuda_buffer import CudaBuffer
from nanoep_b200.types import NativeHandle, NativeLayout


class FakeWorld:
    """all_gather_object / barrier for N threads."""

    def __init__(self, size):
        self.size = size
        self.cond = threading.Condition()
        self.slots = {}
        self.generation = 0
        self.rank_of = {}

    def rank(self):
        return self.rank_of[threading.get_ident()]

    def all_gather_object(self, out, obj, group=None):
        payload = pickle.dumps(obj)
        with self.cond:
            gen = self.generation
            self.slots.setdefault(gen, {})[self.rank()] = payload
            if len(self.slots[gen]) == self.size:
                self.generation += 1
                self.cond.notify_all()
            else:
                assert self.cond.wait_for(lambda: self.generation > gen, timeout=20)
            for r in range(self.size):
                out[r] = pickle.loads(self.slots[gen][r])

    def barrier(self, group=None):
        self.all_gather_object([None] * self.size, None)


class FakeWindow:
    def __init__(self, log, rank, fail_at=None):
        self.log, self.rank, self.fail_at = log, rank, fail_at
        self.log.append((rank, "allocate"))

    def layout(self):
        return {"num_bytes": 4096}

    def export_handle(self):
        if self.fail_at == "export":
            raise OSError("export boom")
        self.log.append((self.rank, "export"))
        return bytes([self.rank]) * 64

    def import_handles(self, handles, peer_devices=()):
        assert [h[0] for h in handles] == list(range(len(handles))) and all(len(h) == 64 for h in handles)
        if self.fail_at == "import":
            raise RuntimeError("import boom")
        self.log.append((self.rank, "import"))

    def close_peer_mappings(self):
        self.log.append((self.rank, "unmap"))

    def close(self):
        self.log.append((self.rank, "free"))


def run_ranks(world, fn):
    results, errors = [None] * world.size, [None] * world.size

    def body(rank):
        world.rank_of[threading.get_ident()] = rank
        try:
            results[rank] = fn(rank)
        except Exception as exc:  # noqa: BLE001
            errors[rank] = exc

    threads = [threading.Thread(target=body, args=(r,)) for r in range(world.size)]
    [t.start() for t in threads]
    [t.join(timeout=30) for t in threads]
    return results, errors


@pytest.fixture
def fake_env(monkeypatch):
    world = FakeWorld(2)
    monkeypatch.setattr(cuda_buffer.dist, "get_world_size", lambda group=None: world.size)
    monkeypatch.setattr(cuda_buffer.dist, "get_rank", lambda group=None: world.rank())
    monkeypatch.setattr(cuda_buffer.dist, "get_backend", lambda group=None: "gloo")
    monkeypatch.setattr(cuda_buffer.dist, "barrier", world.barrier)
    monkeypatch.setattr(bootstrap.dist, "all_gather_object", world.all_gather_object)
    monkeypatch.setattr(bootstrap.dist, "get_world_size", lambda group=None: world.size)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda device=None: None)
    monkeypatch.setattr(torch.cuda, "Stream", lambda device=None: SimpleNamespace(cuda_stream=77))
    monkeypatch.setattr(
        torch.cuda, "get_device_properties",
        lambda device: SimpleNamespace(multi_processor_count=78, uuid=f"GPU-{world.rank()}"),
    )
    monkeypatch.delenv("LOCAL_RANK", raising=False)
    monkeypatch.delenv("LOCAL_WORLD_SIZE", raising=False)
    return world


def test_bootstrap_order_and_close(fake_env, monkeypatch):
    log = []
    monkeypatch.setattr(cuda_buffer, "_load_native", lambda: SimpleNamespace(PeerWindow=lambda rank, *a: FakeWindow(log, rank)))
    cfg = EPConfig(4, 2, 256, 8)

    def body(rank):
        buf = CudaBuffer("group", cfg)
        assert buf.rank == rank and buf.world_size == 2 and buf.comm_stream.cuda_stream == 77
        buf.close()
        buf.close()
        return True

    results, errors = run_ranks(fake_env, body)
    assert errors == [None, None] and results == [True, True]
    for rank in range(2):
        mine = [op for r, op in log if r == rank]
        assert mine == ["allocate", "export", "import", "unmap", "free"]
    # nobody frees before everybody has unmapped
    last_unmap = max(i for i, (_, op) in enumerate(log) if op == "unmap")
    first_free = min(i for i, (_, op) in enumerate(log) if op == "free")
    assert last_unmap < first_free


@pytest.mark.parametrize("fail_at,stage", [("export", "allocation/export"), ("import", "import/stream")])
def test_bootstrap_failure_is_collective_and_rolls_back(fake_env, monkeypatch, fail_at, stage):
    log = []
    monkeypatch.setattr(
        cuda_buffer, "_load_native",
        lambda: SimpleNamespace(PeerWindow=lambda rank, *a: FakeWindow(log, rank, fail_at if rank == 0 else None)),
    )

    def body(rank):
        CudaBuffer("group", EPConfig(4, 2, 256, 8))

    _, errors = run_ranks(fake_env, body)
    assert all(isinstance(e, RuntimeError) for e in errors)
    assert str(errors[0]) == str(errors[1])
    assert str(errors[0]).startswith(f"CudaBuffer {stage} failed: rank 0: ")
    last_unmap = max(i for i, (_, op) in enumerate(log) if op == "unmap")
    first_free = min(i for i, (_, op) in enumerate(log) if op == "free")
    assert last_unmap < first_free
    assert sorted(op for _, op in log if op in ("unmap", "free")) == ["free", "free", "unmap", "unmap"]


def test_environment_validation_messages(fake_env, monkeypatch):
    monkeypatch.setattr(cuda_buffer, "_load_native", lambda: SimpleNamespace(PeerWindow=lambda rank, *a: FakeWindow([], rank)))
    cases = [
        (lambda rank: EPConfig(4, 2, 256, 8 + rank), ValueError, "EPConfig mismatch across ranks"),
        (lambda rank: EPConfig(5, 2, 256, 8), ValueError, "num_experts must be divisible by world_size"),
        (lambda rank: EPConfig(4, 2, 250, 8), ValueError, "hidden must be a positive multiple of 256"),
    ]
    for make_cfg, exc_type, text in cases:
        _, errors = run_ranks(fake_env, lambda rank: CudaBuffer("group", make_cfg(rank)))
        assert all(isinstance(e, exc_type) and str(e) == text for e in errors), errors
    _, errors = run_ranks(fake_env, lambda rank: CudaBuffer("group", EPConfig(4, 2, 256, 8), allow_multiple_reduction=1 if rank else False))
    assert all(isinstance(e, RuntimeError) and "allow_multiple_reduction must be bool" in str(e) for e in errors)


# ---------------------------------------------------------------- dispatch / combine wiring
class FakeBackend:
    def __init__(self):
        self.calls = []

    def dispatch(self, *args):
        self.calls.append(("dispatch", args))
        x = args[1][0]
        K = 2
        meta = [torch.zeros(3, K + 2, dtype=torch.int32), torch.zeros(2, dtype=torch.int64), torch.tensor([0, 2, 4]),
                torch.zeros(x.shape[0], 2, dtype=torch.int64), torch.zeros(2, dtype=torch.int64),
                torch.zeros(x.shape[0], K, dtype=torch.int64), torch.zeros(2, dtype=torch.int64), torch.zeros(4, dtype=torch.int32)]
        cached = args[4][0]
        outputs = [[torch.zeros(4, 256, dtype=torch.bfloat16), torch.zeros(0, dtype=torch.int64), torch.zeros(4)]]
        return outputs, [cached if cached else meta], [(3, 4)], "EVENT" if args[12] else None

    def combine(self, *args):
        self.calls.append(("combine", args))
        return [[torch.zeros(5, 256, dtype=torch.bfloat16), torch.zeros(5, 2)]], "EVENT" if args[11] else None

    @staticmethod
    def HandleState(metadata, capacity, expand):
        return SimpleNamespace(metadata=metadata, capacity=capacity, expand=expand)

    def dispatch_cached(self, *args):
        self.calls.append(("dispatch_cached", args))
        return torch.zeros(4, 256, dtype=torch.bfloat16), torch.zeros(0, dtype=torch.int64), torch.zeros(4), "EVENT" if args[8] else None

    def combine_single(self, *args):
        self.calls.append(("combine_single", args))
        return torch.zeros(5, 256, dtype=torch.bfloat16), torch.zeros(5, 2), "EVENT" if args[9] else None


def make_buffer(monkeypatch):
    buf = CudaBuffer.__new__(CudaBuffer)
    buf._config = EPConfig(4, 2, 256, 8)
    buf._rank, buf._world_size, buf._device, buf._device_sms = 0, 2, 0, 78
    buf._closed, buf._allow_multiple_reduction, buf._auto_num_sms = False, False, None
    buf._backend, buf._window, buf._mailbox_timeout_s = FakeBackend(), "WINDOW", 60.0
    buf._comm_stream = SimpleNamespace(cuda_stream=77)
    buf._gpu_uuids = ("a", "b")
    monkeypatch.setattr(torch.cuda, "device", lambda d: __import__("contextlib").nullcontext())
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    return buf


def test_dispatch_argument_forwarding_and_handles(monkeypatch):
    buf = make_buffer(monkeypatch)
    x = torch.zeros(5, 256, dtype=torch.bfloat16)
    idx = torch.zeros(5, 2, dtype=torch.int64)
    w = torch.zeros(5, 2)
    got = buf.dispatch(x, topk_idx=idx, weights=w)
    name, a = buf._backend.calls[-1]
    assert name == "dispatch" and a[0] == ["WINDOW"] and a[1][0] is x and a[2][0] is idx and a[3][0] is w
    assert a[4] == [[]] and a[5] == [0]
    assert a[6:14] == (1, False, False, 78, 77, -1, False, 60.0)  # alignment 1, compact, no padding, all SMs, sync
    assert got.event is None and got.handle.num_sms == 78 and got.handle.owner is buf
    assert got.handle.layout.recv_count == 3 and got.handle.layout.expanded_capacity == 4 and got.topk_idx is not None
    # expanded + async + explicit budget + previous_event
    ev = SimpleNamespace(cuda_event=1234)
    got2 = buf.dispatch(x, topk_idx=idx, do_expand=True, alignment=16, zero_padding=True, async_op=True, num_sms=12, previous_event=ev)
    a = buf._backend.calls[-1][1]
    assert a[6:13] == (16, True, True, 12, 77, 1234, True)
    assert got2.topk_idx is None and got2.topk_weights is None and got2.event.event == "EVENT"
    assert got2.event.keepalive[0] is buf and got2.event.keepalive[1] is x
    # cached: same handle object; the native state made by the fresh call carries the metadata in the fixed order
    h = got2.handle
    expect = [h.layout.recv_metadata, h.layout.expert_counts, h.layout.expert_offsets, h.dst_slots, h.send_counts, h.topk_idx,
              h.layout.recv_rank_prefix, h.slot_map]
    st = h.native_state
    assert all(u is v for u, v in zip(st.metadata, expect)) and st.capacity == 4 and st.expand is True
    again = buf.dispatch(x, handle=h, weights=w, zero_padding=True, async_op=True)
    name, a = buf._backend.calls[-1]
    assert name == "dispatch_cached" and again.handle is h and again.topk_idx is None and again.event.event == "EVENT"
    assert a[:3] == ("WINDOW", x, w) and a[3] is st and a[4:10] == (True, 12, 77, -1, True, 60.0) and a[10] is None and a[11] == 0
    # a handle without native state (built by hand) takes the list interface: budget and layout inherited
    h.native_state = None
    again = buf.dispatch(x, handle=h, weights=w)
    name, a = buf._backend.calls[-1]
    assert name == "dispatch" and again.handle is h and a[2] == [None] and a[9] == 12 and a[7] is True and a[6] == 16
    assert all(u is v for u, v in zip(a[4][0], expect)) and a[5] == [4]
    h.native_state = st
    # num_sms = 0 -> model (no NVLink information in this process -> all SMs)
    buf.dispatch(x, topk_idx=idx, num_sms=0)
    assert buf._backend.calls[-1][1][9] == 78
    for bad in (dict(num_sms=79), dict(num_sms=-1), dict(num_sms=True), dict(alignment=0), dict(do_expand=1)):
        with pytest.raises(ValueError):
            buf.dispatch(x, topk_idx=idx, **bad)
    with pytest.raises(ValueError):
        buf.dispatch(x)
    with pytest.raises(ValueError):
        buf.dispatch(x, topk_idx=idx, handle=h)
    with pytest.raises(ValueError):
        buf.dispatch(x, handle=h, alignment=4)
    with pytest.raises(ValueError):
        buf.dispatch(torch.zeros(5, 128, dtype=torch.bfloat16), topk_idx=idx)
    buf._closed = True
    with pytest.raises(RuntimeError, match="closed"):
        buf.dispatch(x, topk_idx=idx)


def test_combine_argument_forwarding(monkeypatch):
    buf = make_buffer(monkeypatch)
    layout = NativeLayout(torch.zeros(3, 4, dtype=torch.int32), torch.zeros(2, dtype=torch.int64), torch.tensor([0, 2, 4]),
                          torch.zeros(2, dtype=torch.int64), 3, 4)
    handle = NativeHandle(buf._config, 0, 2, True, 2, torch.zeros(5, 2, dtype=torch.int64), layout, torch.zeros(5, 2, dtype=torch.int64),
                          torch.zeros(2, dtype=torch.int64), buf, torch.bfloat16, num_sms=20, slot_map=torch.zeros(4, dtype=torch.int32))
    monkeypatch.setattr(cuda_buffer, "validate_combine_inputs", lambda *a: None)
    y = torch.zeros(4, 256, dtype=torch.bfloat16)
    out = buf.combine(y, handle, weights=torch.zeros(4), async_op=True)
    name, a = buf._backend.calls[-1]
    assert name == "combine" and a[0] == ["WINDOW"] and a[1][0] is y and a[3] == [4] and a[5] == [None]
    assert a[6:12] == (True, False, 20, 77, -1, True)
    assert out.topk_weights is not None and out.event.keepalive[2] is handle
    handle.native_state = st = FakeBackend.HandleState([], 4, True)
    wts, bias = torch.zeros(4), torch.zeros(5, 256, dtype=torch.bfloat16)
    out = buf.combine(y, handle, weights=wts, bias=bias, async_op=True)
    name, a = buf._backend.calls[-1]
    assert name == "combine_single" and a == ("WINDOW", y, st, wts, bias, False, 20, 77, -1, True)
    assert out.topk_weights is not None and out.event.event == "EVENT" and out.event.keepalive[2] is handle
    other = make_buffer(monkeypatch)
    with pytest.raises(ValueError, match="another"):
        other.combine(y, handle)


def test_determinism_guard(monkeypatch):
    buf = make_buffer(monkeypatch)
    monkeypatch.setattr(torch, "are_deterministic_algorithms_enabled", lambda: True)
    monkeypatch.setattr(cuda_buffer.deterministic, "fill_uninitialized_memory", True)
    with pytest.raises(RuntimeError, match="deterministic"):
        buf.dispatch(torch.zeros(1, 256, dtype=torch.bfloat16), topk_idx=torch.zeros(1, 2, dtype=torch.int64))


def test_peer_access_rules():
    """The rule the window import applies to every mapped peer: a distinct GPU that this GPU can reach."""
    from nanoep_b200.utils.build import load_extension

    ext = load_extension()
    assert ext.peer_access_error(0, 1, 0, 1, True, True) == ""
    same = ext.peer_access_error(2, 3, 5, 5, True, True)
    assert "rank 2" in same and "rank 3" in same and "share CUDA device 5" in same
    for can, supported in ((False, True), (True, False), (False, False)):
        unreachable = ext.peer_access_error(0, 1, 0, 4, can, supported)
        assert "no peer access" in unreachable and "device 4" in unreachable


def test_single_launch_limits_round_trip():
    """The run-time knobs of the single-launch dispatch paths: read, change one, keep the others, restore."""
    from nanoep_b200.utils.build import load_extension

    ext = load_extension()
    before = ext.fused_limits()
    assert len(before) == 3  # (cached dispatch tokens, grid bound, fresh dispatch tokens)
    try:
        ext.set_fused_limits(fresh_tokens=17)
        assert ext.fused_limits() == (before[0], before[1], 17)
        ext.set_fused_limits(dispatch_tokens=5, blocks=9)
        assert ext.fused_limits() == (5, 9, 17)
        ext.set_fused_limits()  # negative / omitted values keep what is there
        assert ext.fused_limits() == (5, 9, 17)
    finally:
        ext.set_fused_limits(*before)
    assert ext.fused_limits() == before


def test_gate_hook_wants_pinned_host_memory():
    import torch

    from nanoep_b200.utils.build import load_extension

    ext = load_extension()
    import pytest

    with pytest.raises(RuntimeError, match="pinned"):
        ext.set_test_gate(torch.zeros(2, dtype=torch.int32), 1.0)  # pageable host memory: the kernel could not poll it
    ext.set_test_gate(None)


def test_combine_shared_memory_plan():
    """The combine's shared-memory plan fits the CTA's limit for every geometry, always leaves the transfer warps a
    ring of at least two stages, keeps chunks 128-byte multiples no longer than a row, and gives up the reduce
    pipeline (register path) rather than the transfer rings when a row is very long."""
    from nanoep_b200.utils.build import load_extension

    ext = load_extension()
    limit = 227 * 1024
    board_and_slack = 4096  # flag board, alignment, mbarriers
    for hidden in (256, 512, 2048, 4096, 7168, 8192, 16384, 32768, 49152):
        for parts in (1, 2, 4, 8, 16, 32):
            for stages in (0, 2, 4):
                warps, ring_stages, smem, r_stages, chunk = ext.combine_plan(hidden, parts, limit, stages, 0)
                pitch = (hidden * 2 + 127) // 128 * 128
                assert 1 <= warps <= 8 and ring_stages in (2, 3), (hidden, parts, stages, warps, ring_stages)
                assert smem + 256 <= limit, (hidden, parts, stages, smem)
                assert smem >= warps * ring_stages * (pitch + 8) + r_stages * parts * chunk
                assert smem <= warps * ring_stages * (pitch + 8) + r_stages * parts * chunk + board_and_slack
                if r_stages:
                    assert r_stages == stages and chunk % 128 == 0 and 128 <= chunk <= pitch
                else:
                    assert chunk == 0
                if stages == 0:
                    assert r_stages == 0
    # the headline geometry: whole-row... two stages of half-row chunks of all eight partitions, four transfer warps
    assert ext.combine_plan(7168, 8, limit, 2, 0) == (4, 2, ext.combine_plan(7168, 8, limit, 2, 0)[2], 2, 7168)
    # a named chunk is rounded up to 128 bytes
    assert ext.combine_plan(7168, 8, limit, 4, 1700)[4] == 1792
    # a row that leaves no room for a pipeline falls back to the register path instead of failing
    assert ext.combine_plan(49152, 8, limit, 2, 0)[3] in (0, 2)
