"""The prequantised-weight sidecar (s2p_qcache.bin): written at the first load, served at the next,
and interchangeable with the reference's in both directions.  A served tensor must be the tensor the
live quantisers produce, so every check ends in identical greedy frames; the two libraries' files are
also compared entry by entry (names, kinds, shapes, lengths and payload bytes)."""
import json
import os
import struct
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def load(which, qdir):
    r = subprocess.run([sys.executable, os.path.join(HERE, "qcache_worker.py"), which, str(qdir)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    served = [l for l in r.stderr.splitlines() if "qcache: serving" in l]
    wrote = [l for l in r.stderr.splitlines() if "qcache: wrote" in l]
    return json.loads(line[7:])["frames"], bool(served), bool(wrote)


def parse(path):
    """name -> (kind, N, K, group, code bytes, scale bytes)"""
    raw = open(path, "rb").read()
    assert raw[:8] == b"S2PQC\x01\x00\x00"
    fingerprint, n = struct.unpack_from("<QI", raw, 8)
    at, out, order = 24, {}, []
    for _ in range(n):
        name_len, kind, N, K, group, _pad, q_off, q_len, s_off, s_len = struct.unpack_from("<IIiiiIQQQQ", raw, at)
        at += 56
        name = raw[at:at + name_len].decode()
        at += name_len
        assert q_off % 256 == 0 and s_off % 256 == 0
        out[name] = (kind, N, K, group, raw[q_off:q_off + q_len], raw[s_off:s_off + s_len])
        order.append(name)
    return fingerprint, out, order


def test_sidecar_round_trip_and_interchange_with_the_reference(tmp_path):
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libs2pref_l2.so")):
        pytest.skip("reference library not built on this machine")
    mine_dir, ref_dir = tmp_path / "mine", tmp_path / "ref"
    mine_dir.mkdir(); ref_dir.mkdir()
    # first load: live quantisers, sidecar written
    f_live, served, wrote = load("mine", mine_dir)
    assert not served and wrote and (mine_dir / "s2p_qcache.bin").exists()
    # second load: served from the sidecar, same frames
    f_served, served, wrote = load("mine", mine_dir)
    assert served and not wrote
    assert f_served == f_live, "tensors served from the sidecar differ from the live quantisers'"
    # the reference writes its own
    r_live, served, wrote = load("ref", ref_dir)
    assert not served and wrote
    assert r_live == f_live
    fp_a, a, order_a = parse(mine_dir / "s2p_qcache.bin")
    fp_b, b, order_b = parse(ref_dir / "s2p_qcache.bin")
    assert fp_a == fp_b, "the staleness fingerprint must be the reference's"
    assert sorted(a) == sorted(b), (sorted(set(a) ^ set(b)))
    for name in a:
        assert a[name][:4] == b[name][:4], name
        assert a[name][4] == b[name][4], f"{name}: quantised codes differ"
        assert a[name][5] == b[name][5], f"{name}: scales differ"
    # each library serves the other's file
    f_from_ref, served, _ = load("mine", ref_dir)
    assert served and f_from_ref == f_live
    r_from_mine, served, _ = load("ref", mine_dir)
    assert served and r_from_mine == r_live
