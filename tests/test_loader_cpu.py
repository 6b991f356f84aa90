"""The C++ weight-container reader (cccc's INIReaderBin format) and its shard-aware loading: each
tensor-parallel rank must read exactly the bytes of its shard.  CPU only."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from __graft_entry__ import load_package
from oracle import oracle as O


def H():
    h = load_package().hostapi
    return h, h.lib()


def tp():
    load_package()
    import importlib

    return importlib.import_module("cccc_lite_b200.tp")


def write_container(path, entries):
    """The container exactly as scripts/convert_weights.py:66-83 lays it out (own code)."""
    index, blobs, off = [], [], 0
    for k, v in entries.items():
        index.append(f"{k} = {off},{len(v)}")
        blobs.append(v)
        off += len(v)
    ini = ("\n".join(index) + "\n").encode("ascii")
    with open(path, "wb") as f:
        f.write(b"CFG_BIN INI" + b"\x00" * 21)
        f.write(struct.pack("<Q", len(ini)))
        f.write(ini)
        f.write(b"".join(blobs))


def load(L, f, name, N, K, kind, world, rank):
    w = np.zeros(N * K * 4, np.uint8)    # room for a float tensor
    s = np.zeros(N * K // 16 + 1, np.uint8)
    qs = C.c_float(0)
    dims = (C.c_int * 3)()
    err = C.create_string_buffer(256)
    rc = L.cccc_host_bin_load_shard(f, name.encode(), N, K, kind.encode(), world, rank, w.ctypes.data, w.size, s.ctypes.data,
                                    s.size, C.byref(qs), dims, err, 256)
    return rc, w, s, qs.value, list(dims), err.value.decode()


@pytest.fixture()
def container(tmp_path):
    N, K = 64, 1024
    W8, _, inv8, _ = O.make_inputs(O.FP8_E5M2, N, K, 1, seed=1, scaled=True)
    W4, blk4, _, _ = O.make_inputs(O.FP4_E2M1, N, K, 1, seed=2)
    legacy = np.array([O.lib().oracle_e4m3_to_float(int(b)) for b in blk4], np.float32)
    path = str(tmp_path / "weights.bin")
    write_container(path, {
        "data_type": b"fp8_e5m2",
        "weight_fp8_e5m2_layers.0.q_proj": W8.tobytes(),
        "scale_layers.0.q_proj": struct.pack("<f", inv8),
        "weight_fp4_e2m1_layers.0.down_proj": W4.tobytes(),
        "blockscale_layers.0.down_proj": blk4.tobytes(),
        "weight_fp4_e2m1_legacy": W4.tobytes(),
        "blockscale_legacy": legacy.tobytes(),
        "weight_bf16_norm": np.zeros(8, np.uint16).tobytes(),
    })
    return path, N, K, (W8, inv8), (W4, blk4)


def test_reads_the_reference_container_and_only_the_shard_bytes(container):
    path, N, K, (W8, inv8), (W4, blk4) = container
    h, L = H()
    T = tp()
    f = L.cccc_host_bin_open(path.encode())
    assert f and L.cccc_host_bin_has(f, b"data_type") and not L.cccc_host_bin_has(f, b"nope")
    for world in (1, 2, 4):
        for rank in range(world):
            for kind in ("c", "r"):
                before = L.cccc_host_bin_bytes_read(f)
                rc, w, s, qs, dims, err = load(L, f, "layers.0.q_proj", N, K, kind, world, rank)
                assert rc == 0, err
                sh = T.make_shard("col" if kind == "c" else "row", N, K, world, rank, O.FP8_E5M2)
                want, _ = T.slice_weight(W8, None, sh, N, K, O.FP8_E5M2)
                assert dims == [O.FP8_E5M2, sh.N, sh.K] and np.float32(qs) == np.float32(inv8)
                assert np.array_equal(w[:want.size], want)
                # bytes fetched from the file: the shard and the 4-byte scale, nothing else
                assert L.cccc_host_bin_bytes_read(f) - before == want.size + 4
                if world * 256 <= K:
                    rc, w, s, qs, dims, err = load(L, f, "layers.0.down_proj", N, K, kind, world, rank)
                    assert rc == 0, err
                    sh = T.make_shard("col" if kind == "c" else "row", N, K, world, rank, O.FP4_E2M1)
                    want, wants = T.slice_weight(W4, blk4, sh, N, K, O.FP4_E2M1)
                    assert dims == [O.FP4_E2M1, sh.N, sh.K] and qs == 1.0
                    assert np.array_equal(w[:want.size], want) and np.array_equal(s[:wants.size], wants)
    # legacy float32 block scales are re-encoded to E4M3 on load
    rc, w, s, qs, dims, err = load(L, f, "legacy", N, K, "c", 2, 1)
    assert rc == 0 and np.array_equal(s[:N * K // 32], blk4.reshape(N, K // 16)[N // 2:].reshape(-1))
    L.cccc_host_bin_close(f)


def test_loader_refuses_bad_requests(container, tmp_path):
    path, N, K, _, _ = container
    h, L = H()
    f = L.cccc_host_bin_open(path.encode())
    for args, word in ((("missing", N, K, "c", 1, 0), "not found"), (("norm", 2, 5, "c", 1, 0), "N*K"),
                       (("layers.0.q_proj", N + 1, K, "c", 1, 0), "N*K"), (("layers.0.q_proj", N, K, "c", 3, 0), "divide"),
                       (("layers.0.q_proj", N, K, "r", 32, 0), "k steps"), (("layers.0.down_proj", N, K, "r", 8, 0), "k steps"),
                       (("layers.0.q_proj", N, K, "x", 1, 0), "kind"), (("layers.0.q_proj", N, K, "c", 2, 2), "rank")):
        rc, *_, err = load(L, f, *args)
        assert rc == -1 and word in err, (args, err)
    L.cccc_host_bin_close(f)
    # truncated file, bad magic, missing file
    data = open(path, "rb").read()
    t = str(tmp_path / "trunc.bin")
    open(t, "wb").write(data[:len(data) // 2])
    assert not L.cccc_host_bin_open(t.encode())
    open(t, "wb").write(b"NOT A BIN" + data[9:])
    assert not L.cccc_host_bin_open(t.encode())
    assert not L.cccc_host_bin_open(str(tmp_path / "absent.bin").encode())


def test_unquantised_tensors_load_as_raw_shards(tmp_path):
    """BF16 / float checkpoints (quantised on the GPU after loading): a column shard is a run of rows, a row shard
    one run per row, in the tensor's own element type."""
    h, L = H()
    N, K = 8, 1024
    rng = np.random.default_rng(5)
    Wb = rng.integers(0, 1 << 16, (N, K)).astype(np.uint16)
    Wf = rng.standard_normal((N, K)).astype(np.float32)
    path = str(tmp_path / "raw.bin")
    write_container(path, {"weight_bf16_a": Wb.tobytes(), "weight_float_b": Wf.tobytes()})
    f = L.cccc_host_bin_open(path.encode())
    for name, W, dt in (("a", Wb, O.BFLOAT16), ("b", Wf, O.FLOAT)):
        for world in (1, 2, 4):
            for rank in range(world):
                rc, w, _, qs, dims, err = load(L, f, name, N, K, "c", world, rank)
                want = W[rank * N // world:(rank + 1) * N // world]
                assert rc == 0 and dims == [dt, N // world, K] and qs == 1.0, err
                assert w[:want.nbytes].tobytes() == want.tobytes()
                rc, w, _, qs, dims, err = load(L, f, name, N, K, "r", world, rank)
                want = np.ascontiguousarray(W[:, rank * K // world:(rank + 1) * K // world])
                assert rc == 0 and dims == [dt, N, K // world], err
                assert w[:want.nbytes].tobytes() == want.tobytes()
    rc, *_, err = load(L, f, "a", N, K, "r", 8, 0)
    assert rc == -1 and "k steps" in err
    L.cccc_host_bin_close(f)


def test_writer_round_trip(tmp_path):
    h, L = H()
    keys = [b"a", b"weight_fp8_e5m2_w", b"empty"]
    blobs = [b"hello", bytes(range(256)) * 4, b""]
    path = str(tmp_path / "out.bin")
    karr = (C.c_char_p * 3)(*keys)
    barr = (C.c_void_p * 3)(*[C.cast(C.create_string_buffer(b, len(b)), C.c_void_p) if b else None for b in blobs])
    larr = (C.c_ulonglong * 3)(*[len(b) for b in blobs])
    assert L.cccc_host_bin_write(path.encode(), 3, karr, barr, larr) == 0
    raw = open(path, "rb").read()
    assert raw[:11] == b"CFG_BIN INI" and raw[11:32] == b"\x00" * 21
    n = struct.unpack("<Q", raw[32:40])[0]
    assert raw[40:40 + n].decode() == "a = 0,5\nweight_fp8_e5m2_w = 5,1024\nempty = 1029,0\n"
    assert raw[40 + n:] == b"".join(blobs)
    f = L.cccc_host_bin_open(path.encode())
    rc, w, s, qs, dims, err = load(L, f, "w", 4, 256, "c", 2, 1)
    assert rc == 0 and np.array_equal(w[:512], np.frombuffer(blobs[1], np.uint8)[512:])
    L.cccc_host_bin_close(f)


@pytest.mark.parametrize("dtype,suffix", [(O.FP8_E5M2, "fp8_e5m2"), (O.FP8_E4M3, "fp8_e4m3"), (O.FP4_E2M1, "fp4_e2m1")])
def test_quantised_tensors_are_written_under_the_loaders_keys(tmp_path, dtype, suffix):
    """BinWriter::addQuantised: weight_<dtype>_<name>, scale_<name> (FP8) or blockscale_<name> (FP4), read back by the
    shard loader bit for bit."""
    h, L = H()
    N, K = 16, 512
    rng = np.random.default_rng(dtype)
    wbytes = N * K // 2 if dtype == O.FP4_E2M1 else N * K
    W = rng.integers(0, 256, wbytes).astype(np.uint8)
    S = rng.integers(0, 120, N * K // 16).astype(np.uint8) if dtype == O.FP4_E2M1 else None
    path = str(tmp_path / "q.bin")
    rc = L.cccc_host_bin_write_quantised(path.encode(), b"W_q_0", dtype, N, K, W.ctypes.data, W.size, S.ctypes.data if S is not None else None,
                                         S.size if S is not None else 0, 0.37)
    assert rc == 0
    f = L.cccc_host_bin_open(path.encode())
    assert L.cccc_host_bin_has(f, f"weight_{suffix}_W_q_0".encode())
    assert bool(L.cccc_host_bin_has(f, b"scale_W_q_0")) == (dtype != O.FP4_E2M1)
    assert bool(L.cccc_host_bin_has(f, b"blockscale_W_q_0")) == (dtype == O.FP4_E2M1)
    rc, w, s, qs, dims, err = load(L, f, "W_q_0", N, K, "c", 1, 0)
    assert rc == 0 and dims == [dtype, N, K], err
    assert np.array_equal(w[:wbytes], W)
    if dtype == O.FP4_E2M1:
        assert np.array_equal(s[:S.size], S)
    else:
        assert np.float32(qs) == np.float32(0.37)
    L.cccc_host_bin_close(f)
