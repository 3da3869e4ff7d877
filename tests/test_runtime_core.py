"""The C++ runtime library: SBP geometry vs the Python twin, control store (KV, barrier time-out, heartbeat
failure detection — all failures are produced on the host), caching allocator, persistent table, executor
ordering, record / token readers."""
import os
import subprocess
import sys
import threading
import time

import numpy as np
import pytest

import oneflow as flow
from oneflow_b200 import runtime as R
from oneflow_b200.framework.balanced_splitter import BalancedSplitter
from oneflow_b200.framework import nd_sbp


def test_sbp_geometry_matches_python():
    S, B, P = flow.sbp.split, flow.sbp.broadcast, flow.sbp.partial_sum
    for total, parts in [(10, 4), (7, 7), (3, 5), (128, 8)]:
        for i in range(parts):
            assert R.balanced_split(total, parts, i) == BalancedSplitter(total, parts).at(i)
    for nd in [(S(0), S(0)), (S(1), B), (B, S(0)), (P, S(2))]:
        for c in [(0, 0), (1, 2), (1, 0)]:
            assert R.slice_view((9, 7, 5), (2, 3), nd, c) == nd_sbp.slice_view((9, 7, 5), (2, 3), nd, c)
    for a in (S(0), S(1), B, P):
        for b in (S(0), S(1), B, P):
            assert abs(R.copy_cost(a, b, 1000.0, 4) - nd_sbp.copy_cost(a, b, 1000.0, 4)) < 1e-9


def test_control_store_kv_barrier_and_timeouts():
    srv = R.ControlServer(world_size=3)
    cs = [R.ControlClient("127.0.0.1", srv.port, r) for r in range(3)]
    cs[0].set("nccl_id", b"\x01\x02\x03")
    assert cs[2].get("nccl_id") == b"\x01\x02\x03"
    assert cs[1].add("cnt", 5) == 5 and cs[2].add("cnt", 2) == 7
    with pytest.raises(TimeoutError):
        cs[1].get("never-set", timeout_s=0.2)
    done = []
    ths = [threading.Thread(target=lambda c=c: (c.barrier("b0", 3, 5.0), done.append(1))) for c in cs]
    [t.start() for t in ths]
    [t.join() for t in ths]
    assert len(done) == 3
    # one rank skips the barrier (ranks executing different code): the others get a time-out, not a hang
    t0 = time.time()
    with pytest.raises(TimeoutError) as ei:
        cs[0].barrier("b1", 3, 0.3)
    assert time.time() - t0 < 3 and "different code" in str(ei.value)
    for c in cs:
        c.close()
    srv.stop()


def test_heartbeat_detects_a_rank_that_stops():
    srv = R.ControlServer(world_size=3)
    cs = [R.ControlClient("127.0.0.1", srv.port, r) for r in range(3)]
    for c in cs:
        c.start_heartbeat(0.05)
    time.sleep(0.3)
    assert cs[0].lost_ranks(0.5) == []
    cs[2].close()                 # rank 2 "dies" between steps (host side only)
    time.sleep(0.7)
    assert cs[0].lost_ranks(0.5) == [2] and cs[1].lost_ranks(0.5) == [2]
    cs[0].close()
    cs[1].close()
    srv.stop()


def test_bin_allocator_host_backend():
    a = R.BinAllocator("host", chunk_bytes=1 << 20)
    p1, p2, p3 = a.alloc(1000), a.alloc(300000), a.alloc(5000)
    assert len({p1, p2, p3}) == 3 and p1 % 512 == 0
    st = a.stats()
    assert st["chunks"] == 1 and st["in_use"] == 1024 + 300032 + 5120
    a.free(p2)
    p4 = a.alloc(200000)          # best fit: reuses the hole left by p2
    assert p4 == p2
    big = a.alloc(3 << 20)        # larger than a chunk: gets its own chunk
    assert a.stats()["chunks"] == 2
    for p in (p1, p3, p4, big):
        a.free(p)
    with pytest.raises(R.core.CoreError):
        a.free(p1)                # double free is reported
    assert a.stats()["in_use"] == 0 and a.stats()["free_blocks"] == 2   # fully coalesced
    assert a.shrink() == 2 and a.stats()["reserved"] == 0
    a.destroy()


def test_persistent_table_roundtrip_and_snapshots(tmp_path):
    t = R.PersistentTable(tmp_path / "tbl", value_bytes=24 * 4, block_bytes=512)
    keys = np.array([5, 1 << 40, 7, 9], dtype=np.int64)
    vals = np.random.rand(4, 24).astype(np.float32)
    t.put(keys, vals)
    got, found = t.get(np.array([7, 6, 5], dtype=np.int64))
    assert found.tolist() == [True, False, True] and np.allclose(got[0], vals[2]) and np.all(got[1] == 0)
    t.save_snapshot("s1")
    t.put(np.array([6, 7], dtype=np.int64), np.ones((2, 24), np.float32))
    assert len(t) == 5
    assert np.allclose(t.get(np.array([7], np.int64))[0][0], 1.0)      # the live table sees the update
    t.save_snapshot("s2")
    t.load_snapshot("s1")
    # a snapshot is point-in-time: key 7 reads the value it had when s1 was taken, key 6 does not exist yet
    assert len(t) == 4 and not t.get(np.array([6], np.int64))[1][0]
    assert np.allclose(t.get(keys)[0], vals)
    # writing on after loading the older snapshot must not disturb the rows of the younger one
    t.put(np.array([11], dtype=np.int64), np.full((1, 24), 3.0, np.float32))
    t.load_snapshot("s2")
    assert len(t) == 5 and np.allclose(t.get(np.array([6, 7], np.int64))[0], 1.0)
    t.load_snapshot("s1")
    t.close()
    t2 = R.PersistentTable(tmp_path / "tbl", value_bytes=24 * 4)   # index persisted on close
    assert len(t2) == 4 and np.allclose(t2.get(keys)[0], vals)
    t2.close()


def test_persistent_table_index_survives_a_session_that_never_closed(tmp_path):
    t = R.PersistentTable(tmp_path / "tbl", value_bytes=8 * 4, block_bytes=512)
    keys = np.arange(10, dtype=np.int64)
    vals = np.random.rand(10, 8).astype(np.float32)
    t.put(keys, vals)
    # no close(): the index file was never written, only the put log
    t2 = R.PersistentTable(tmp_path / "tbl", value_bytes=8 * 4, block_bytes=512)
    assert len(t2) == 10 and np.allclose(t2.get(keys)[0], vals)
    t2.close()
    t.close()


def test_executor_respects_dependencies_and_overlaps_streams():
    ex = R.TaskExecutor(n_streams=3)
    log, lock = [], threading.Lock()

    def task(name, dur):
        def f():
            time.sleep(dur)
            with lock:
                log.append(name)
        return f
    ex.submit(0, task("w1", 0.10), writes=[1])
    ex.submit(1, task("r1a", 0.01), reads=[1])        # after w1
    ex.submit(2, task("r1b", 0.01), reads=[1])        # after w1, concurrently with r1a
    ex.submit(0, task("w1_again", 0.01), writes=[1])  # after both readers
    ex.submit(1, task("free", 0.0), writes=[2])       # independent object, same stream as r1a: stays behind it
    ex.wait_all(10)
    assert log.index("w1") < log.index("r1a") and log.index("w1") < log.index("r1b")
    assert log.index("w1_again") > max(log.index("r1a"), log.index("r1b"))
    assert log.index("free") > log.index("r1a") and ex.completed() == 5
    t0 = time.time()
    for s in range(3):
        ex.submit(s, task(f"p{s}", 0.2), writes=[100 + s])
    ex.wait_all(10)
    assert time.time() - t0 < 0.5                      # three streams in parallel, not 0.6 s
    ex.destroy()


def test_record_and_token_readers(tmp_path):
    recs = [bytes([i]) * (i + 1) for i in range(50)]
    R.write_records(tmp_path / "r.bin", recs)
    assert list(R.RecordReader(tmp_path / "r.bin")) == recs
    shuffled = list(R.RecordReader(tmp_path / "r.bin", shuffle_buffer=16, seed=3))
    assert sorted(shuffled) == sorted(recs) and shuffled != recs
    toks = np.arange(1000, dtype=np.uint16)
    toks.tofile(tmp_path / "t.bin")
    ds = R.TokenDataset(tmp_path / "t.bin", token_bytes=2)
    assert len(ds) == 1000
    b = ds.batch([0, 3], seq_len=8)
    assert b.shape == (2, 9) and b[1].tolist() == list(range(24, 33))
    with pytest.raises(R.core.CoreError):
        ds.batch([200], seq_len=8)
    ds.close()


def test_record_reader_reports_corrupt_and_truncated_files(tmp_path):
    """A length prefix larger than the rest of the file, or a file that ends inside a record, is an error the
    caller sees (not a crash of the reader thread and not a silent end of data)."""
    import struct
    good = [b"abc", b"defgh"]
    R.write_records(tmp_path / "ok.bin", good)
    raw = (tmp_path / "ok.bin").read_bytes()
    (tmp_path / "huge.bin").write_bytes(raw + struct.pack("<Q", 1 << 60) + b"xy")
    r = R.RecordReader(tmp_path / "huge.bin")
    assert next(r) == b"abc" and next(r) == b"defgh"
    with pytest.raises(R.CoreError, match="corrupt length prefix"):
        next(r)
    r.close()
    (tmp_path / "cut.bin").write_bytes(raw[:-2])            # payload cut short: its prefix now exceeds the file
    r = R.RecordReader(tmp_path / "cut.bin")
    assert next(r) == b"abc"
    with pytest.raises(R.CoreError, match="corrupt length prefix"):
        next(r)
    r.close()
    (tmp_path / "cut2.bin").write_bytes(raw[:len(raw) - 5 - 3])   # the file ends inside the second length prefix
    r = R.RecordReader(tmp_path / "cut2.bin")
    assert next(r) == b"abc"
    with pytest.raises(R.CoreError, match="ends inside a record"):
        next(r)
    r.close()


def test_host_runtime_selftest_under_sanitizers(tmp_path):
    """The multi-threaded self-test of the host runtime (executor ordering over a non-atomic counter, concurrent allocator
    use, store clients with heartbeats, table writers with snapshots, the record prefetch thread) runs clean under
    ThreadSanitizer and under AddressSanitizer + UBSan."""
    import subprocess
    from oneflow_b200 import build as B
    exes = B.build_sanitizers()
    assert len(exes) == 2
    for exe in exes:
        d = tmp_path / os.path.basename(exe)
        d.mkdir()
        env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66", ASAN_OPTIONS="detect_leaks=1 exitcode=67")
        r = subprocess.run([exe, str(d)], capture_output=True, text=True, timeout=600, env=env)
        out = r.stdout + r.stderr
        assert r.returncode == 0, out[-3000:]
        assert "core selftest ok" in out
        assert "ThreadSanitizer" not in out and "AddressSanitizer" not in out and "runtime error" not in out, out[-3000:]
