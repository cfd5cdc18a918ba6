"""GEAR's loader / sampler / copy API on the GPU through the mirrors, checked against the
oracle: next(loader) must return the bytes the oracle gathers for the indices the sampler
reports, for uniform and weighted sampling, host-mapped and HBM-resident tables."""
import numpy as np
import pytest
import torch

import gear_b200.dropin

gear_b200.dropin.install()

import gear  # noqa: E402
import libgear.core as glibc  # noqa: E402
from gear.dataset import SharedDataset  # noqa: E402
from gear.loader import OfflineLoader  # noqa: E402
from gear.mpu import ModelParallelismUnit  # noqa: E402
from gear.specs import TableSpec  # noqa: E402

pytestmark = pytest.mark.gpu


def test_reference_test_copy():
    # tests/test_copy.py of the reference, verbatim in meaning
    device = torch.device("cuda:0")
    column_shapes = (4, 3, 2)
    data = torch.ones((32, 100) + column_shapes, dtype=torch.float32, device="cpu", pin_memory=True)
    copied = torch.zeros((10,) + column_shapes, dtype=torch.float32, device=device)
    src_offset = torch.zeros(1, dtype=torch.long, device=device)
    dst_offset = torch.zeros(1, dtype=torch.long, device=device)
    stride = copied.numel() * copied.element_size() * torch.ones(1, dtype=torch.long, device=device)
    glibc.copy_debug(data, copied, src_offset, dst_offset, stride, stride[0])
    torch.cuda.synchronize()
    assert torch.all(copied)


def _dataset(O, cap, T, key, residency):
    spec = TableSpec.create(0, 1, T, cap, [dict(shape=[17], dtype=torch.float32, name="obs"),
                                           dict(shape=[6], dtype=torch.float32, name="act"),
                                           dict(shape=[], dtype=torch.float32, name="rew"),
                                           dict(shape=[], dtype=torch.uint8, name="done")])
    ds = SharedDataset.create(spec, create=True, key=key, residency="host")
    rng = np.random.default_rng(key)
    for i in range(cap):
        cols = [torch.from_numpy(rng.standard_normal((T, 17)).astype(np.float32)),
                torch.from_numpy(rng.uniform(-1, 1, (T, 6)).astype(np.float32)),
                torch.from_numpy(rng.standard_normal(T).astype(np.float32)),
                torch.from_numpy((np.arange(T) == T - 1).astype(np.uint8))]
        ds[i] = (float(rng.lognormal()), int(rng.integers(1, T + 1)), cols)
    if residency == "hbm":
        ds.to_hbm()
    return ds


@pytest.mark.parametrize("residency", ["host", "hbm"])
@pytest.mark.parametrize("method", ["Uniform", "Weighted"])
def test_offline_loader_matches_oracle(O, residency, method):
    gear.init(0)
    cap, T, B, L = 64, 50, 32, 20
    ds = _dataset(O, cap, T, key=7000 + len(residency) + len(method), residency=residency)
    mpu = ModelParallelismUnit(device=torch.device("cuda:0"), dp_rank=0, dp_world_size=1)
    pats = [dict(name="obs", offset=-L, length=L, pad="head"), dict(name="act", offset=-L, length=L, pad="head"),
            dict(name="done", offset=-3, length=5, pad="tail")]
    loader = OfflineLoader(ds, B, mpu, method, pats)
    img = np.array(ds._table._t.host_view(), copy=True)
    rows = [68, 24, 4, 1]
    accu, stride = O.table_layout(rows, T)
    for _ in range(3):
        tss, data = next(loader)
        torch.cuda.synchronize()
        # the sampler's last draw, sorted, is what the loader gathered
        idx = torch.sort(loader._indices[loader._sampler._cache]).values.cpu().numpy()
        lens = ds.timesteps.numpy()[idx]
        assert np.array_equal(tss.cpu().numpy(), lens)
        assert list(data[0].shape) == [B, L, 17] and data[0].dtype == torch.float32 and data[2].dtype == torch.uint8
        for out, (col, off, ln, head) in zip(data, [(0, -L, L, True), (1, -L, L, True), (3, -3, 5, False)]):
            want = O.fused_subcopy(img, idx, lens, lens, stride, int(accu[col]), T, rows[col], off, ln, head)
            assert np.array_equal(out.cpu().numpy().view(np.uint8).reshape(-1), want)
    if method == "Weighted":
        # same variates => same indices as the oracle's search on the same weights
        w = ds.weights.numpy().astype(np.float32)
        ocdf, ol1, _, _ = O.scan(w)
        u = O.philox_u01(42, loader._sampler._calls - 1, 0, B)
        assert np.array_equal(np.sort(O.search(ocdf, ol1, u, scale=True)), idx)
    # the two-step route (host sub + vcopy) gives the same tensors as the fused one
    sel = torch.arange(0, cap, 3)
    fused = loader.exposed_fused_iterate(sel)
    _, two_step = loader.exposed_low_level_controlled_iterate(sel)
    torch.cuda.synchronize()
    for a, b in zip(fused, two_step):
        assert torch.equal(a, b)


def test_weighted_draw_with_replacement_gives_duplicate_rows(O):
    # The reference's WeightedSampler calls torch.multinomial with its default replacement=False
    # (gear/sampler/global_sampler.py:170): a batch never holds an index twice, and a batch larger
    # than the number of candidates with weight raises.  Here the draw is with replacement (it
    # consumes external variates), so a batch larger than the table is served and some trajectories
    # appear in several rows; every row, duplicates included, holds that trajectory's bytes.
    gear.init(0)
    cap, T, B, L = 8, 30, 32, 6
    ds = _dataset(O, cap, T, key=7100, residency="hbm")
    with pytest.raises(RuntimeError):
        torch.multinomial(ds.weights.float().cuda(), B)            # what the reference's call would do
    mpu = ModelParallelismUnit(device=torch.device("cuda:0"), dp_rank=0, dp_world_size=1)
    loader = OfflineLoader(ds, B, mpu, "Weighted", [dict(name="obs", offset=0, length=L, pad="tail")])
    img = np.array(ds._table._t.host_view(), copy=True)
    accu, stride = O.table_layout([68, 24, 4, 1], T)
    tss, data = next(loader)
    torch.cuda.synchronize()
    idx = torch.sort(loader._indices[loader._sampler._cache]).values.cpu().numpy()
    assert len(np.unique(idx)) < B                                  # pigeonhole: 32 draws from 8 trajectories
    lens = ds.timesteps.numpy()[idx]
    want = O.fused_subcopy(img, idx, lens, lens, stride, int(accu[0]), T, 68, 0, L, False)
    got = data[0].cpu().numpy().view(np.uint8).reshape(B, -1)
    assert np.array_equal(got.reshape(-1), want)
    for i in range(1, B):
        if idx[i] == idx[i - 1]:
            assert np.array_equal(got[i], got[i - 1])


def test_checkpoint_of_an_hbm_table_above_2_gib_streams_both_ways(tmp_path):
    # A table that exists in device memory only, larger than 2 GiB (where the reference's pickle
    # stops: it holds the table as one bytes object and casts its size to int on load,
    # src/storage/pybind.cc:178-204), is written chunk by chunk through a pinned bounce buffer
    # and read back straight into HBM.  Compared chunk by chunk on the device.
    import shutil
    from gear_b200 import _native as N
    from gear_b200 import core
    gear.init(0)
    T, cap = 1000, 550                                   # 550 x 1000 x 4100 B = 2.255 GB > 2 GiB
    need = cap * T * 4100
    if shutil.disk_usage(tmp_path).free < need + (1 << 30):
        pytest.skip("not enough room for a 2.3 GB checkpoint in the temporary directory")
    spec = TableSpec.create(0, 1, T, cap, [dict(shape=[1024], dtype=torch.int32, name="obs"),
                                           dict(shape=[], dtype=torch.float32, name="rew")])
    ds = SharedDataset.create(spec, create=True, key=7300, residency="hbm")
    t = ds._table._t
    assert t.nbytes == need > (1 << 31) and not t.host_ptr
    core.fill_ptr(t.device_ptr, t.nbytes // 4, N.FILL_U32, seed=0x5EED)
    ds.weights[:] = torch.arange(cap, dtype=torch.float32)
    ds.timesteps[:] = T
    path = tmp_path / "big.ckpt"
    ds.checkpoint(path)                                  # HBM only: streamed by default
    assert path.stat().st_size > need
    back = SharedDataset().load(path, key=7301)          # lands where it was: HBM only
    tb = back._table._t
    assert tb.nbytes == need and not tb.host_ptr and tb.device_ptr and tb.device_ptr != t.device_ptr
    a = core.device_view(t.device_ptr, need // 8, torch.int64)
    b = core.device_view(tb.device_ptr, need // 8, torch.int64)
    chunk = (64 << 20) // 8
    for off in range(0, need // 8, chunk):
        x, y = a[off:off + chunk], b[off:off + chunk]
        assert int(x.sum()) == int(y.sum()) and torch.equal(x[::4097], y[::4097]), off
    assert torch.equal(a, b)
    assert torch.equal(back.weights, ds.weights)
    # and the loader's gather works on the reloaded table
    mpu = ModelParallelismUnit(device=torch.device("cuda:0"), dp_rank=0, dp_world_size=1)
    loader = OfflineLoader(back, 8, mpu, "Uniform", [dict(name="obs", offset=0, length=4, pad="tail")])
    tss, data = next(loader)
    torch.cuda.synchronize()
    assert list(data[0].shape) == [8, 4, 1024]
