"""Batch sources: the row choice against the reference's own ``get_activations`` (CPU) and the device
gathers against plain indexing (GPU)."""
import multiprocessing as mp
import types
from multiprocessing import shared_memory

import pytest
import torch

from crosslayer_transcoder_b200 import data
from oracle import ref_import


class FakeStore:
    """The attributes of the reference's SharedActivationBuffer that a consumer touches
    (crosslayer_transcoder/data/shared_memory.py:62-121), over real POSIX shared memory."""

    def __init__(self, n, L, D, dtype=torch.float16, threshold=0.0, batch_size=None):
        self.buffer_size, self.minimum_fill_threshold, self.batch_size = n, threshold, batch_size
        shape = (n, 2, L, D)
        nel = n * 2 * L * D
        self.shm = shared_memory.SharedMemory(create=True, size=nel * torch.empty((), dtype=dtype).element_size())
        self.buffer_tensor = torch.frombuffer(self.shm.buf, dtype=dtype, count=nel).view(shape)
        self.validity_tensor = torch.zeros(n, dtype=torch.bool)
        self.buffer_lock, self.validity_lock = mp.RLock(), mp.RLock()
        self.stats = {"total_reads": 0, "last_read_time": None}

    def fill(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.buffer_tensor.copy_(torch.randn(self.buffer_tensor.shape, generator=g))
        self.buffer_tensor[:, 0, 0, 0] = torch.arange(self.buffer_size, dtype=torch.float32)   # row id, exact in fp16
        self.validity_tensor.fill_(True)

    def close(self):
        del self.buffer_tensor
        self.shm.close()
        self.shm.unlink()


@pytest.fixture
def store():
    s = FakeStore(96, 3, 64)
    s.fill()
    yield s
    s.close()


def test_draw_rows_respects_threshold_and_count(store):
    store.validity_tensor[10:] = False
    with store.buffer_lock:
        assert data.draw_rows(store, 11) is None                      # fewer valid rows than asked for
        rows = data.draw_rows(store, 10)
    assert sorted(rows.tolist()) == list(range(10))
    store.minimum_fill_threshold = 0.5
    with store.buffer_lock:
        assert data.draw_rows(store, 4) is None                       # below the fill threshold
    data.retire_rows(store, rows[:4])
    assert int(store.validity_tensor.sum()) == 6 and store.stats["total_reads"] == 1


def test_draw_rows_match_reference_get_activations(store):
    """Same seed, same store state: the reference's own method returns exactly the rows draw_rows picks,
    and leaves the same validity mask behind."""
    ref = ref_import.load_shared_memory()
    if ref is None:
        pytest.skip("reference sources not present")
    cls = ref.SharedActivationBuffer
    store.validity_tensor[::3] = False
    before = store.validity_tensor.clone()
    for name in ("get_activations", "_get_valid_indices", "_mark_indices_invalid"):    # unmodified methods
        setattr(store, name, types.MethodType(getattr(cls, name), store))
    torch.manual_seed(7)
    want = store.get_activations(16)
    after_ref = store.validity_tensor.clone()
    store.validity_tensor.copy_(before)
    torch.manual_seed(7)
    with store.buffer_lock:
        rows = data.draw_rows(store, 16)
    assert torch.equal(store.buffer_tensor[rows], want)
    data.retire_rows(store, rows)
    assert torch.equal(store.validity_tensor, after_ref)


def _ids(batch):
    return batch[:, 0, 0, 0].float().cpu().long()


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["mapped", "staged"])
def test_shared_buffer_batches(store, mode):
    src = data.SharedBufferBatches(store, batch_size=8, device="cuda:0", depth=2, mode=mode)
    try:
        seen = []
        for _ in range(5):
            b = next(src)
            assert b.is_cuda and b.shape == (8, 2, 3, 64)
            ids = _ids(b)
            assert torch.equal(b.cpu(), store.buffer_tensor[ids])      # whole rows, bit-exact
            seen += ids.tolist()
        assert len(set(seen)) == len(seen)                             # a row is handed out once
        assert not store.validity_tensor[seen].any()
        src.gather.check()
    finally:
        src.close()
    # the batch in flight at close() was retired too; nothing else was touched
    assert int((~store.validity_tensor).sum()) == 6 * 8


@pytest.mark.gpu
def test_shared_buffer_batches_wait_for_refill_and_time_out(store):
    store.validity_tensor.fill_(False)
    src = data.SharedBufferBatches(store, batch_size=8, device="cuda:0", timeout=0.3)
    try:
        with pytest.raises(TimeoutError):
            next(src)
    finally:
        src.close()
    src = data.SharedBufferBatches(store, batch_size=8, device="cuda:0", timeout=30.0)
    try:
        with store.buffer_lock:                                        # a producer fills 8 rows
            store.validity_tensor[40:48] = True
        assert sorted(_ids(next(src)).tolist()) == list(range(40, 48))
        assert not store.validity_tensor.any()                         # nothing left to prefetch: no gather in flight
        with store.buffer_lock:
            store.validity_tensor[8:16] = True
        assert sorted(_ids(next(src)).tolist()) == list(range(8, 16))
    finally:
        src.close()
    with pytest.raises(ValueError):
        data.SharedBufferBatches(store, batch_size=0, device="cuda:0")


@pytest.mark.gpu
@pytest.mark.parametrize("resident", [True, False])
def test_tensor_batches_follow_reference_order(resident):
    g = torch.Generator().manual_seed(3)
    t = torch.randn(50, 2, 3, 64, generator=g).half()
    src = data.TensorBatches(t, 16, shuffle=True, device="cuda:0", resident=resident)
    torch.manual_seed(11)
    it = iter(src)
    got = [next(it).clone() for _ in range(9)]
    torch.manual_seed(11)
    want = []
    while len(want) < 9:                          # InfiniteTensorDataset.__iter__ (tensor_datamodule.py:22-34)
        idx = torch.randperm(50)
        want += [t[idx[i:i + 16]] for i in range(0, 50, 16)]
    for a, b in zip(got, want):
        assert a.shape == b.shape and torch.equal(a.cpu(), b)
    src.gather.check()
    src.close()


@pytest.mark.gpu
def test_tensor_datamodule_and_bad_rows(tmp_path):
    t = torch.arange(40 * 2 * 2 * 8, dtype=torch.float32).view(40, 2, 2, 8)
    torch.save(t, tmp_path / "acts.pt")
    dm = data.TensorDataModule(str(tmp_path / "acts.pt"), batch_size=16, shuffle=False, device="cuda:0")
    dm.setup("fit")
    it = iter(dm.train_dataloader())
    assert torch.equal(next(it).cpu(), t[:16]) and torch.equal(next(it).cpu(), t[16:32])
    assert torch.equal(next(it).cpu(), t[32:]) and torch.equal(next(it).cpu(), t[:16])
    gth = dm.dataset.gather
    ev = gth.launch(0, torch.tensor([1, 40, 2]))                      # row 40 does not exist: skipped, reported
    ev.synchronize()
    with pytest.raises(Exception, match="out of range"):
        gth.check()
    dm.teardown()


@pytest.mark.gpu
def test_training_step_consumes_store_batches():
    """A module trains directly from the batches the device-side consumer yields: same loss as the same rows
    indexed on the host and uploaded."""
    from crosslayer_transcoder_b200 import synthetic
    from tests.helpers import build_module, spec_inputs

    spec = synthetic.WorkloadSpec("ingest", 3, 64, 256, 32, "jumprelu", True, False, rank_u=8, n_outlier=1,
                                  lambda_sparsity=1e-4, pre_actv_loss=3e-6, lr=1e-3)
    batch, w, la = spec_inputs(spec)
    s = FakeStore(128, spec.n_layers, spec.d_acts)
    try:
        g = torch.Generator().manual_seed(2)
        s.buffer_tensor.copy_(torch.randn(s.buffer_tensor.shape, generator=g))
        s.buffer_tensor[:, 0, 0, 0] = torch.arange(128, dtype=torch.float32)
        s.validity_tensor.fill_(True)
        dev = torch.device("cuda:0")
        mod = build_module(spec, w, dev)
        twin = build_module(spec, w, dev)
        src = data.SharedBufferBatches(s, batch_size=spec.batch, device="cuda:0")
        try:
            for i in range(2):
                b = next(src)
                ids = _ids(b)
                loss = mod.training_step(b, i)
                want = twin.training_step(s.buffer_tensor[ids].to(dev), i)
                assert abs(float(loss) - float(want)) <= 1e-6 * abs(float(want))
                loss.backward()
                want.backward()
            mod._engine.check_status("ingest")
        finally:
            src.close()
    finally:
        s.close()
