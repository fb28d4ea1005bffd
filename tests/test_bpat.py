"""`.bpat` files: header/index parsing and checksum verification run on the CPU; loading into device
tensors and writing are GPU tests.  Fixtures come from an independent Python encoder
(tests/golden/make_bpat_fixtures.py) that follows the reference's documented layouts
(crates/fused_gpu/src/io/headers.rs:16-117)."""
import json
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_bpat_fixtures as fx  # noqa: E402

GOLD = os.path.join(HERE, "golden")
FORMATS = {"v0": 0, "v1": 1, "v1m": 2, "v2": 3, "v2f16": 4, "v2bf16": 5}


@pytest.mark.parametrize("fmt", list(FORMATS))
def test_inspect_fixture(fmt):
    from ferrograd_b200 import bpat
    path = os.path.join(GOLD, f"fixture_{fmt}.bpat")
    assert open(path, "rb").read() == fx.encode(fmt, fx.tensors())      # the committed file is what the script makes
    shapes, code = bpat.inspect(path)
    assert code == FORMATS[fmt]
    assert shapes == [(3, 5), (7,), (2, 3, 4)]


@pytest.mark.parametrize("fmt", ["v1", "v1m"])
def test_checksums_are_verified(tmp_path, fmt):
    from ferrograd_b200 import FgError, bpat
    good = fx.encode(fmt, fx.tensors())
    for pos in (20, len(good) // 2, len(good) - 1):       # shape/data, data, the file checksum itself
        bad = bytearray(good)
        bad[pos] ^= 0x40
        p = tmp_path / f"bad_{pos}.bpat"
        p.write_bytes(bytes(bad))
        with pytest.raises(FgError):
            bpat.inspect(p)


def test_truncated_and_foreign_files_are_rejected(tmp_path):
    from ferrograd_b200 import FgError, bpat
    good = fx.encode("v2", fx.tensors())
    (tmp_path / "short.bpat").write_bytes(good[:-10])
    (tmp_path / "other.bpat").write_bytes(b"NOTBPAT!" + good[8:])
    for name in ("short.bpat", "other.bpat", "missing.bpat"):
        with pytest.raises(FgError):
            bpat.inspect(tmp_path / name)


def test_reference_example_checkpoint_summary():
    # data/v2f32_readme.bpat of the reference: five weight tensors of its README example.
    from ferrograd_b200 import bpat
    s = json.load(open(os.path.join(GOLD, "bpat_reference_readme_summary.json")))
    assert s["shapes"] == [[768, 512], [512, 384], [256, 768], [384, 256], [256, 256]]
    assert s["bytes"] == 9 + sum(4 + 8 + 4 * a * b for a, b in s["shapes"])
    ref = os.path.join(os.environ.get("FERROGRAD_REFERENCE", ""), "data", "v2f32_readme.bpat")
    if os.environ.get("FERROGRAD_REFERENCE") and os.path.exists(ref):      # only where the reference tree is at hand
        shapes, code = bpat.inspect(ref)
        assert code == 3 and [list(x) for x in shapes] == s["shapes"]


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", list(FORMATS))
def test_load_fixture_to_device(fmt):
    from ferrograd_b200 import GpuContext, bpat  # noqa: F401
    ctx = GpuContext.new()
    try:
        got = ctx.load_tensors(os.path.join(GOLD, f"fixture_{fmt}.bpat"))
        for t, ref in zip(got, fx.tensors()):
            assert t.shape == ref.shape
            if fmt == "v2f16":
                assert t.dtype == np.float16 and np.array_equal(ctx.to_numpy(t), ref.astype(np.float16))
            elif fmt == "v2bf16":
                assert np.array_equal(ctx.to_numpy(t), fx.bf16_bits(ref))          # bf16 bit patterns
            else:
                assert np.array_equal(ctx.to_numpy(t), ref)      # f64 files hold f32-representable values
    finally:
        ctx.destroy()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,header", [("v2", 3), ("v1m", 2)])
def test_save_is_byte_identical_and_round_trips(tmp_path, fmt, header):
    from ferrograd_b200 import FgError, GpuContext, bpat  # noqa: F401
    ctx = GpuContext.new()
    try:
        ts = [ctx.init_tensor_f32(a.shape, a) for a in fx.tensors()]
        p = tmp_path / f"out_{fmt}.bpat"
        ctx.save_tensors(p, ts, header)
        assert p.read_bytes() == fx.encode(fmt, fx.tensors())
        back = ctx.load_tensors(p)
        for t, ref in zip(back, fx.tensors()):
            assert np.array_equal(ctx.to_numpy(t), ref)
        with pytest.raises(FgError):
            ctx.save_tensors(tmp_path / "x.bpat", ts, 0)     # v0 cannot be written
    finally:
        ctx.destroy()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,header", [("v2f16", 4), ("v2bf16", 5)])
def test_save_16bit_is_byte_identical_and_round_trips(tmp_path, fmt, header):
    # io/headers.rs:60-98: the same layout as v2-f32 with 2-byte elements; 16-bit tensors in, 16-bit tensors out
    from ferrograd_b200 import FgError, GpuContext, bpat  # noqa: F401
    ctx = GpuContext.new()
    try:
        if fmt == "v2f16":
            ts = [ctx.init_tensor_f16(a.shape, a.astype(np.float16)) for a in fx.tensors()]
        else:
            ts = [ctx.init_tensor_bf16(a.shape, a) for a in fx.tensors()]
        p = tmp_path / f"out_{fmt}.bpat"
        ctx.save_tensors(p, ts, header)
        assert p.read_bytes() == fx.encode(fmt, fx.tensors())
        back = ctx.load_tensors(p)
        for t, src in zip(back, ts):
            assert np.array_equal(ctx.to_numpy(t).view(np.uint16), ctx.to_numpy(src).view(np.uint16))
        f32 = [ctx.init_tensor_f32(a.shape, a) for a in fx.tensors()]
        with pytest.raises(FgError):
            ctx.save_tensors(tmp_path / "x.bpat", f32, header)   # f32 tensors do not fit a 16-bit file
    finally:
        ctx.destroy()


@pytest.mark.gpu
def test_trainer_checkpoint_resumes_bit_for_bit(tmp_path):
    """Parameters in the reference's v2-f32 format, AdamW moments and step count in the sidecar container
    (not a reference format): a run resumed from them continues exactly as the uninterrupted run does."""
    from ferrograd_b200 import GpuContext, bpat, dp
    from ferrograd_b200.mlp import MLPTrainer
    dims, batch = [96, 160, 10], 192
    opt = ("adamw", 1e-3, 0.9, 0.999, 1e-8, 0.01)
    wl = dict(dims=dims, batch=batch, loss="ce")
    ctx = GpuContext(0)
    try:
        def run(tr, first, last):
            for s in range(first, last):
                tr.upload_batch(*dp.synth_batch(wl, 0, s, batch))
                tr.step()
            ctx.sync()

        a = MLPTrainer(ctx, dims, batch, "gelu", "ce", opt)
        a.set_params(*MLPTrainer.init_params(dims, "he_normal", 9))
        run(a, 0, 3)
        path = tmp_path / "net.bpat"
        a.save_checkpoint(path)
        shapes, fmt = bpat.inspect(path)
        assert fmt == bpat.V2_F32 and shapes == [(96, 160), (160,), (160, 10), (10,)]
        m, v, step = bpat.load_adamw_state(ctx, str(path) + ".adamw")
        assert step == 3 and [t.shape for t in m] == shapes and [t.shape for t in v] == shapes
        for t in m + v:
            t.data.free()
        run(a, 3, 6)
        Wa, ba = a.get_params()

        b = MLPTrainer(ctx, dims, batch, "gelu", "ce", opt)
        b.load_checkpoint(path)
        run(b, 3, 6)
        Wb, bb = b.get_params()
        for x, y in zip(Wa + ba, Wb + bb):
            assert np.array_equal(x, y)
        with pytest.raises(ValueError):
            bpat.load_adamw_state(ctx, path)            # a parameter file is not a state container (even count)
    finally:
        ctx.sync()
        ctx.destroy()
