"""GEAR's Python-facing API on top of this build, without a GPU: the reference's own spec
tests (tests/test_specs.py:10-34) run unchanged against the mirror, plus dataset
create / write / checkpoint / load and the host-side `sub` through the loader's route."""
import pickle as pkl

import numpy as np
import pytest
import torch

import gear_b200.dropin

gear_b200.dropin.install()

import gear  # noqa: E402
import libgear.core as glibc  # noqa: E402
from gear.dtypes import CVT_DTYPES_GEAR_TO_TORCH as CVT_GTT  # noqa: E402
from gear.specs import ColumnSpec, TableSpec  # noqa: E402


@pytest.mark.parametrize(
    "shape, dtype, name",
    [
        ((3,), torch.bool, "bool"),
        ((3, 4), torch.uint8, "uint8"),
        ((3, 4, 5), torch.int8, "int8"),
        ((3, 4, 5, 6), torch.int32, "int32"),
        ((3, 4, 5, 6, 7), torch.int64, "int64"),
        ((3, 4, 5, 6, 7, 8), torch.float32, "float32"),
        ((3, 4, 5, 6, 7, 8, 9), torch.float64, "float64"),
    ],
)
class TestColumnSpec:
    def test_column_spec_build(self, shape, dtype, name):
        cspec = ColumnSpec.create(shape, dtype, name)
        assert tuple(cspec.shape) == shape
        assert CVT_GTT[cspec.dtype] == dtype
        assert cspec.name == name

    def test_column_spec_pickle(self, shape, dtype, name):
        cspec = ColumnSpec.create(shape, dtype, name)
        cspec_recoverd = pkl.loads(pkl.dumps(cspec))
        assert cspec.shape == cspec_recoverd.shape
        assert cspec.dtype == cspec_recoverd.dtype
        assert cspec.name == cspec_recoverd.name


def test_modules_are_aliases_not_copies():
    import gear_b200.gear.specs as ours
    assert gear.specs is ours and glibc is gear_b200.libgear.core


def test_dtype_names_and_sizes():
    assert glibc.short is glibc.int16 and glibc.long is glibc.int64 and glibc.float is glibc.float32
    assert glibc.ColumnSpec([17], glibc.float32, "obs").size() == 68
    assert glibc.ColumnSpec([4, 84, 84], glibc.uint8, "frames").size() == 28224
    with pytest.raises(RuntimeError):
        glibc.ColumnSpec([2], glibc.half, "h").size()            # sizeof_dtype has no half (dtypes.h:61-73)
    with pytest.raises(RuntimeError):
        glibc.TableSpec(0, 1, 10, 4, 2, [glibc.ColumnSpec([1], glibc.int32, "a")])


def _spec(cap=6, T=20):
    return TableSpec.create(0, 1, T, cap, [dict(shape=[17], dtype=torch.float32, name="obs"),
                                           dict(shape=[6], dtype=torch.float32, name="act"),
                                           dict(shape=[], dtype=torch.float32, name="rew"),
                                           dict(shape=[], dtype=torch.uint8, name="done")])


def test_dataset_write_view_checkpoint_load(tmp_path):
    from gear.dataset import SharedDataset
    spec = _spec()
    assert spec.size() == 97 * 20 * 6 and spec.index("rew") == 2 and spec.index("nope") == -1
    key = 0x51A0 + (id(spec) % 1000)
    ds = SharedDataset.create(spec, create=True, key=key)
    g = torch.Generator().manual_seed(0)
    cols = {}
    for i in range(6):
        c = [torch.randn(20, 17, generator=g), torch.rand(20, 6, generator=g) * 2 - 1, torch.randn(20, generator=g),
             (torch.arange(20) == 19).to(torch.uint8)]
        cols[i] = c
        ds[i] = (float(i + 1), 20 - i, c)
    e = ds[3]
    assert float(e.weight) == 4.0 and int(e.timestep) == 17
    assert torch.equal(e.column0, cols[3][0]) and torch.equal(e.column3, cols[3][3])
    path = tmp_path / "ckpt" / "ds.pkl"
    ds.checkpoint(path)
    ds2 = SharedDataset().load(path, key=key + 1)
    assert torch.equal(ds2.weights, ds.weights) and torch.equal(ds2.timesteps, ds.timesteps)
    for i in range(6):
        for c in range(4):
            assert torch.equal(ds2.get_tensor_view(i)[c], cols[i][c])
    # host-side sub through the handler, reference argument order (handler.cc:78-131)
    h = ds2._handler
    h.set([0], [glibc.SubscribePattern(-5, 5, glibc.SubscribePattern.PadOption.head)])
    idx = torch.tensor([0, 5]); ts = ds2.timesteps[idx]
    s, d, b = (torch.zeros(2, dtype=torch.long) for _ in range(3))
    slot = h.sub(glibc.Int64Span.from_tensor(idx), glibc.Int64Span.from_tensor(ts), glibc.Int64Span.from_tensor(ts), 0,
                 glibc.Int64Span.from_tensor(s), glibc.Int64Span.from_tensor(d), glibc.Int64Span.from_tensor(b))
    assert slot == 5 * 68
    assert s.tolist() == [0 * 1940 + 15 * 68, 5 * 1940 + 10 * 68] and b.tolist() == [340, 340] and d.tolist() == [0, 340]
    with pytest.raises(RuntimeError, match="without setting its SubscribePattern"):
        h.sub(idx, ts, ts, 1, s, d, b)


def test_subscribe_pattern_pickle_and_repr():
    p = glibc.SubscribePattern(-3, 7, glibc.SubscribePattern.PadOption.head)
    q = pkl.loads(pkl.dumps(p))
    assert (q.offset, q.length, q.pad_option) == (-3, 7, glibc.SubscribePattern.PadOption.head)
    assert "kHead" in repr(q) and glibc.SubscribePattern(0, 1).pad_option == glibc.SubscribePattern.PadOption.tail


def test_sub_outputs_write_through_or_are_refused():
    # handler.sub fills caller-owned offset arrays (handler.cc:78-131); an output the results could
    # not reach -- a non-contiguous tensor, which would have to be copied first -- is refused.
    import libgear.core as glibc
    spec = TableSpec.create(0, 1, 10, 4, [dict(shape=[3], dtype=torch.float32, name="x")])
    table = glibc.TrajectoryTable(spec, 0, True)
    table.connect()
    h = glibc.get_cpu_handler(table, 4, glibc.Range(0, 4), glibc.Range(0, 4))
    h.set([0], [glibc.SubscribePattern(0, 2, glibc.SubscribePattern.PadOption.tail)])
    idx, ts, ln = torch.tensor([1, 3]), torch.tensor([0, 9]), torch.tensor([10, 10])
    s, d, b = (torch.zeros(2, dtype=torch.int64) for _ in range(3))
    assert h.sub(idx, ts, ln, 0, s, d, b) == 24
    assert s.tolist() == [120, 3 * 120 + 9 * 12] and d.tolist() == [0, 24] and b.tolist() == [24, 12]
    wide = torch.zeros(2, 2, dtype=torch.int64)
    with pytest.raises(RuntimeError):
        h.sub(idx, ts, ln, 0, wide[:, 0], d, b)
    with pytest.raises(RuntimeError):
        glibc.Int64Span.from_tensor(wide[:, 0])


def test_streamed_checkpoint_round_trip_and_corruption(tmp_path):
    # The table written as header + raw chunks + CRC-32 per chunk (several chunks here), read back
    # by the same load() that reads the reference-style pickle; a flipped byte is caught.
    from gear.dataset import SharedDataset
    import libgear.core as glibc
    spec = TableSpec.create(0, 1, 20, 6, [dict(shape=[5], dtype=torch.float32, name="x"),
                                          dict(shape=[], dtype=torch.uint8, name="d")])
    ds = SharedDataset.create(spec, create=True, key=9100)
    rng = np.random.default_rng(1)
    for i in range(6):
        ds[i] = (float(i + 1), 20 - i, [torch.from_numpy(rng.standard_normal((20, 5)).astype(np.float32)),
                                        torch.from_numpy(rng.integers(0, 255, 20).astype(np.uint8))])
    img = np.array(ds._table._t.host_view(), copy=True)
    glibc.TrajectoryTable.STREAM_CHUNK = 1000            # 2,520 bytes -> three chunks
    try:
        for streamed in (True, False):
            path = tmp_path / f"ckpt_{int(streamed)}.pkl"
            ds.checkpoint(path, streamed=streamed)
            back = SharedDataset().load(path, key=9200 + int(streamed))
            assert np.array_equal(back._table._t.host_view(), img)
            assert torch.equal(back.weights, ds.weights) and torch.equal(back.timesteps, ds.timesteps)
        raw = bytearray((tmp_path / "ckpt_1.pkl").read_bytes())
        raw[len(raw) // 2] ^= 0x40
        (tmp_path / "bad.pkl").write_bytes(bytes(raw))
        with pytest.raises(RuntimeError, match="CRC-32"):
            SharedDataset().load(tmp_path / "bad.pkl", key=9300)
    finally:
        glibc.TrajectoryTable.STREAM_CHUNK = 64 << 20
