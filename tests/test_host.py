"""Host-side pieces that need no GPU: the MPI stand-in, the launcher, the profile-file reader/writer, and
the serving executable's refusal to run without a GPU."""
import ctypes as C
import json
import os
import subprocess

import pytest

from conftest import ROOT

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def host_bins(liger):
    liger.build_all()
    liger.build.build_host()
    return liger.build


@pytest.fixture(scope="module")
def shim_check(host_bins, tmp_path_factory):
    out = str(tmp_path_factory.mktemp("shim") / "mpi_shim_check")
    shim_dir = os.path.join(ROOT, "24ppopp-liger_b200", "host", "mpi_shim")
    subprocess.run(["g++", "-O2", "-std=c++17", "-I", shim_dir, "-o", out, os.path.join(HERE, "mpi_shim_check.cc"),
                    os.path.join(shim_dir, "mpi_shim.cc"), "-lrt", "-lpthread"], check=True)
    return out


@pytest.mark.parametrize("np_", [1, 2, 4])
def test_mpi_shim_bcast_and_barrier(host_bins, shim_check, np_):
    env = dict(os.environ, LIGER_MPI_TIMEOUT_S="60")
    res = subprocess.run([host_bins.MPIRUN_PATH, "-np", str(np_), shim_check], capture_output=True, text=True, timeout=120,
                         env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    lines = [l for l in res.stdout.splitlines() if " ok " in l]
    assert len(lines) == np_
    assert len({l.split(" ok ")[1] for l in lines}) == 1   # every rank saw the same broadcast stream


def test_mpi_shim_reports_a_missing_rank_instead_of_hanging(host_bins, shim_check):
    """Failure detection on the host: a rank that never joins makes the others give up with an error."""
    env = dict(os.environ, LIGER_MPI_RANK="0", LIGER_MPI_SIZE="2", LIGER_MPI_JOB=f"lonely{os.getpid()}",
               LIGER_MPI_TIMEOUT_S="2")
    res = subprocess.run([shim_check], capture_output=True, text=True, timeout=60, env=env)
    assert res.returncode == 3
    assert "timeout" in res.stderr


def test_launcher_propagates_failure(host_bins):
    res = subprocess.run([host_bins.MPIRUN_PATH, "-np", "2", "/bin/sh", "-c", "exit $LIGER_MPI_RANK"], timeout=30)
    assert res.returncode == 1


def test_serving_executable_fails_loudly_without_a_gpu(host_bins):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    res = subprocess.run([host_bins.MAIN_PATH, "2", "64", "4", "64", "1", "7", "2", "100", "--mode", "no_schedule"],
                         capture_output=True, text=True, timeout=60)
    assert res.returncode != 0
    assert "GPU" in res.stderr or "CUDA" in res.stderr


def test_profile_files_round_trip(liger, tmp_path):
    lib = liger.lib()
    main = [{"kernel_name": k, "batch_size": 2, "seq_len": s, "duration": 0.125 * (k + 1) + s * 1e-3}
            for k in range(7) for s in (16, 32, 48)]
    sub = [{"kernel_name": k, "batch_size": 2, "seq_len": 32, "duration": [0.01 * i * (k + 1) for i in range(1, 8)]}
           for k in (0, 2, 3, 4, 5, 6)]
    for name, data, is_sub in (("Main.json", main, 0), ("Sub.json", sub, 1)):
        src, dst = tmp_path / name, tmp_path / ("out_" + name)
        src.write_text(json.dumps(data))
        n, tot = C.c_int(0), C.c_double(0)
        liger.check(lib.liger_profile_rewrite(str(src).encode(), str(dst).encode(), is_sub, C.byref(n), C.byref(tot)))
        assert n.value == len(data)
        want = sum(sum(e["duration"]) if is_sub else e["duration"] for e in data)
        assert tot.value == pytest.approx(want, rel=1e-5)
        back = json.loads(dst.read_text())          # what the library writes is valid JSON in the same schema
        key = lambda e: (e["kernel_name"], e["batch_size"], e["seq_len"])
        assert sorted(map(key, back)) == sorted(map(key, data))
        for e in back:
            ref = next(d for d in data if key(d) == key(e))
            assert e["duration"] == pytest.approx(ref["duration"], rel=1e-5)


def test_profile_reader_accepts_the_reference_writers_spelling(liger, tmp_path):
    """src/utils.h:160-188 writes `"duration": [a,b,...]` with a space after the colon and no other whitespace."""
    p = tmp_path / "Sub_ref.json"
    p.write_text('[{"kernel_name":0,"batch_size":2,"seq_len":64,"duration": [0.1,0.2,0.3]},'
                 '{"kernel_name":8,"batch_size":2,"seq_len":64,"duration": [1e-05,2.5]}]')
    n, tot = C.c_int(0), C.c_double(0)
    liger.check(liger.lib().liger_profile_rewrite(str(p).encode(), None, 1, C.byref(n), C.byref(tot)))
    assert n.value == 2 and tot.value == pytest.approx(3.10001, rel=1e-5)


@pytest.mark.parametrize("text", ["", "[", '[{"kernel_name":0}]', '[{"kernel_name":0,"batch_size":1,"seq_len":4,"duration":}]',
                                  '{"kernel_name":0}', '[{"kernel_name":0,"batch_size":1,"seq_len":4,"duration":[1,2]}]'])
def test_malformed_profile_is_an_error(liger, tmp_path, text):
    p = tmp_path / "bad.json"
    p.write_text(text)
    assert liger.lib().liger_profile_rewrite(str(p).encode(), None, 0, None, None) == -1
    assert b"profile" in liger.lib().liger_last_error()


def test_empty_profile_is_valid(liger, tmp_path):
    """The reference's writer produces invalid JSON for an empty dictionary (src/utils.h:117); "[]" here."""
    p, q = tmp_path / "empty.json", tmp_path / "empty_out.json"
    p.write_text("[]")
    n = C.c_int(-1)
    liger.check(liger.lib().liger_profile_rewrite(str(p).encode(), str(q).encode(), 0, C.byref(n), None))
    assert n.value == 0 and json.loads(q.read_text()) == []


def test_missing_profile_file_is_an_error(liger):
    assert liger.lib().liger_profile_rewrite(b"/nonexistent/Main.json", None, 0, None, None) == -1


def test_cost_model_interpolates_between_profiled_shapes(liger, tmp_path):
    """The scheduler's cost model (liger_profile_predict) serves every (batch, length) from a profile taken at a few
    lengths; the reference's lookup returns 0 for anything it did not profile (src/schedule.h:166)."""
    lib = liger.lib()
    main = [{"kernel_name": 4, "batch_size": 8, "seq_len": s, "duration": 0.2 + s * 0.01} for s in (128, 256, 512)]
    main += [{"kernel_name": 100, "batch_size": 0, "seq_len": 0, "duration": 0.06}]      # a measured contention factor
    p = tmp_path / "Main.json"
    p.write_text(json.dumps(main))

    def predict(name, bs, sq):
        out = C.c_double(-1.0)
        liger.check(lib.liger_profile_predict(str(p).encode(), 16, 1024, name, bs, sq, C.byref(out)))
        return out.value

    assert predict(4, 8, 256) == pytest.approx(0.2 + 2.56, rel=1e-6)                    # profiled
    assert predict(4, 8, 192) == pytest.approx(0.2 + 1.92, rel=1e-6)                    # between 128 and 256: linear
    assert predict(4, 8, 300) == pytest.approx(0.2 + 3.00, rel=1e-6)
    assert predict(4, 8, 64) == pytest.approx(0.2 + 1.28, rel=1e-6)                     # below the first: its value, a floor
    assert predict(4, 8, 1024) == pytest.approx((0.2 + 5.12) * 2.0, rel=1e-6)           # beyond the last: in proportion
    assert predict(4, 4, 256) == pytest.approx((0.2 + 2.56) * 0.5, rel=1e-6)            # other batch size: by tokens
    assert predict(4, 16, 192) == pytest.approx((0.2 + 1.92) * 2.0, rel=1e-6)
    assert predict(5, 8, 256) == 0.0                                                    # never profiled
    assert lib.liger_profile_predict(None, 16, 1024, 4, 8, 256, None) == -1


def test_few_row_gemm_plan_covers_every_k_block_once(liger):
    """The host-side choice between the two few-row GEMM kernels (liger_gemm_smallm_plan; no GPU involved).
    For the stream-K kernel the plan is `per` k-blocks per CTA over the tile-major line of (tile, k-block) pairs:
    replaying the kernel's own arithmetic, every k-block of every tile is covered exactly once, a CTA hands over
    at most two partial tiles (its first and its last) into distinct slots, and the contributors the last arrival
    sums for a tile are exactly the CTAs that touched it.  For the cluster kernel the splits cover K and the
    grid is tiles x splits.  And at the shapes of a GLM-130B decode step the long-K / few-tile weights
    (out-projection and FFN-down at TP = 1) go to stream-K, the TP = 8 QKV weight to a single wave of clusters."""
    lib = liger.lib()

    def plan(n, k, sm):
        out = (C.c_int * 4)()
        assert lib.liger_gemm_smallm_plan(n, k, sm, out) == 0
        return list(out)

    import random
    rnd = random.Random(7)
    cases = [(12288, 12288, 148), (12288, 32768, 148), (36864, 12288, 148), (65536, 12288, 148), (4608, 12288, 148),
             (12288, 1536, 148), (1096, 1024, 148), (8, 8, 148), (38400, 2560, 148)]
    cases += [(8 * rnd.randint(1, 6000), 8 * rnd.randint(1, 3000), rnd.choice([148, 132, 16])) for _ in range(300)]
    seen = set()
    for (n, k, sm) in cases:
        kernel, splits, per, ctas = plan(n, k, sm)
        tiles, kblocks = -(-n // 128), -(-k // 64)
        seen.add(kernel)
        if kernel == 2:
            assert 1 <= splits <= 8 and splits <= kblocks and ctas == tiles * splits and per * splits >= kblocks
            continue
        assert kernel == 3 and splits == 1 and ctas <= sm and ctas == -(-tiles * kblocks // per)
        covered, slots, touched = {}, set(), {}
        for c in range(ctas):
            u, end, parts = c * per, min((c + 1) * per, tiles * kblocks), 0
            assert u < end
            while u < end:
                t = u // kblocks
                lo = u - t * kblocks
                hi = min(kblocks, lo + end - u)
                covered.setdefault(t, []).append((lo, hi))
                if not (lo == 0 and hi == kblocks):
                    slot = 2 * c + (1 if t != (c * per) // kblocks else 0)
                    assert slot not in slots
                    slots.add(slot)
                    touched.setdefault(t, []).append(c)
                    parts += 1
                u += hi - lo
            assert parts <= 2
        for t in range(tiles):
            segs = sorted(covered[t])
            assert segs[0][0] == 0 and segs[-1][1] == kblocks and all(a[1] == b[0] for a, b in zip(segs, segs[1:]))
            first, last = (t * kblocks) // per, ((t + 1) * kblocks - 1) // per
            assert touched.get(t, [first]) == list(range(first, last + 1)) or (t not in touched and first == last)
    assert seen == {2, 3}
    assert plan(12288, 12288, 148)[0] == 3 and plan(12288, 32768, 148)[0] == 3     # long K, 96 tiles
    assert plan(4608, 12288, 148)[:2] == [2, 4] or plan(4608, 12288, 148)[:2] == [2, 3]   # one wave of clusters
    assert lib.liger_gemm_smallm_plan(0, 64, 148, (C.c_int * 4)()) < 0
