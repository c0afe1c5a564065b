"""CPU-only checks: the C ABI library loads and exports everything the header
declares, and the host-side pieces (Matrix Market I/O, conversion, partitioner)
behave like the reference code they replace."""
import os
import re

import numpy as np
import pytest

import oracle
from sddmm_gpu_b200 import api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "sddmm_b200.h")).read()
    declared = sorted(set(re.findall(r"SDDMM_API\s+[\w\s\*]+?\b(sddmm_\w+)\s*\(", header)))
    assert declared, "no declarations parsed"
    L = api.lib()
    for name in declared:
        assert hasattr(L, name), f"{name} declared in the header but not exported"
    assert sorted(declared) == sorted(api.EXPORTED_SYMBOLS)


def test_status_strings():
    L = api.lib()
    seen = {L.sddmm_status_string(i) for i in range(12)}
    assert len(seen) == 12 and b"unknown status" not in seen
    assert L.sddmm_status_string(99) == b"unknown status"


def test_no_gpu_means_no_device_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(api.SddmmError) as e:
        api.Handle(0)
    assert e.value.status == api.NO_DEVICE


def write(tmp_path, text, name="m.mtx"):
    p = tmp_path / name
    p.write_text(text)
    return str(p)


def test_mtx_reader_accepts_what_the_reference_accepts(tmp_path):
    text = ("%%MatrixMarket matrix coordinate real general\n% a comment\n%\n"
            "3 4 5\n1 1 1.5\n1 4 2\n2 2 -3e0\n3 1 4\n3 3 5.25\n")
    M, N, rows, cols, vals = api.mtx_read(write(tmp_path, text))
    assert (M, N) == (3, 4)
    assert list(rows) == [0, 0, 1, 2, 2] and list(cols) == [0, 3, 1, 0, 2]
    assert list(vals) == [1.5, 2.0, -3.0, 4.0, 5.25]
    assert api.coo_is_row_sorted(rows)


def test_mtx_reader_extras_and_errors(tmp_path):
    # size line first (the reference cannot parse this), pattern field, blank lines
    M, N, rows, cols, vals = api.mtx_read(write(tmp_path, "2 2 2\n1 1 7\n2 2 8\n"))
    assert (M, N, list(vals)) == (2, 2, [7.0, 8.0])
    M, N, rows, cols, vals = api.mtx_read(write(tmp_path, "%%MatrixMarket matrix coordinate pattern general\n\n2 3 2\n1 3\n2 1\n"))
    assert list(vals) == [1.0, 1.0] and list(cols) == [2, 0]
    for bad, status in [
        ("%%MatrixMarket matrix coordinate real general\n2 2 2\n1 1\n2 2\n", api.PARSE_ERROR),   # no value column
        ("%%MatrixMarket matrix coordinate real general\n2 2 3\n1 1 1\n2 2 1\n", api.PARSE_ERROR),  # truncated
        ("%%MatrixMarket matrix coordinate real general\n2 2 1\n3 1 1\n", api.INDEX_OUT_OF_RANGE),
        ("%%MatrixMarket matrix coordinate real general\n2 2 1\n0 1 1\n", api.INDEX_OUT_OF_RANGE),
        ("%%MatrixMarket matrix array real general\n2 2\n1\n2\n3\n4\n", api.PARSE_ERROR),
        ("% only comments\n", api.PARSE_ERROR),
        ("%%MatrixMarket matrix coordinate real general\nx y z\n", api.PARSE_ERROR),
    ]:
        with pytest.raises(api.SddmmError) as e:
            api.mtx_read(write(tmp_path, bad))
        assert e.value.status == status, bad
    with pytest.raises(api.SddmmError) as e:
        api.mtx_read(str(tmp_path / "missing.mtx"))
    assert e.value.status == api.IO_ERROR


def test_mtx_round_trip(tmp_path):
    rng = np.random.default_rng(1)
    M, N, nnz = 40, 30, 200
    cells = np.sort(rng.choice(M * N, nnz, replace=False))
    rows, cols = (cells // N).astype(np.int32), (cells % N).astype(np.int32)
    vals = rng.standard_normal(nnz).astype(np.float32)
    path = str(tmp_path / "rt.mtx")
    api.mtx_write(path, M, N, rows, cols, vals)
    M2, N2, r2, c2, v2 = api.mtx_read(path)
    assert (M2, N2) == (M, N)
    assert np.array_equal(r2, rows) and np.array_equal(c2, cols) and np.array_equal(v2, vals)


def test_conversion_matches_reference_converter():
    g = np.load(os.path.join(ROOT, "tests", "golden", "convert.npz"))
    M, N = int(g["M"]), int(g["N"])
    m2, n2, r, c, v = api.coo_sort_rows(M, N, g["rows_in"], g["cols_in"], g["vals_in"], transpose=True)
    # the reference writes 1-based indices of the transpose (util.h:105-107)
    assert (m2, n2) == (N, M)
    assert np.array_equal(r + 1, g["rows_out"]) and np.array_equal(c + 1, g["cols_out"])
    assert np.array_equal(v, g["vals_out"])
    # and against the oracle's restatement on a fresh input
    rng = np.random.default_rng(4)
    cells = rng.choice(60 * 45, 500, replace=False)
    rows, cols = (cells // 45).astype(np.int32), (cells % 45).astype(np.int32)
    vals = rng.standard_normal(500).astype(np.float32)
    ro, co, vo, _, n = oracle.cpu.unsorted_make_csr(rows, cols, vals, 60, 45, True)
    _, _, r, c, v = api.coo_sort_rows(60, 45, rows, cols, vals, transpose=True)
    assert n == 500 and np.array_equal(r + 1, ro) and np.array_equal(c + 1, co) and np.array_equal(v, vo)


def test_plain_row_sort_is_stable_and_keeps_wide_matrices_whole():
    rng = np.random.default_rng(5)
    M, N, nnz = 20, 300, 900   # N > M: the reference's converter would drop entries here
    cells = rng.choice(M * N, nnz, replace=False)
    rows, cols = (cells // N).astype(np.int32), (cells % N).astype(np.int32)
    vals = np.arange(nnz, dtype=np.float32)
    m2, n2, r, c, v = api.coo_sort_rows(M, N, rows, cols, vals, transpose=False)
    order = np.lexsort((cols, rows))
    assert (m2, n2) == (M, N)
    assert np.array_equal(r, rows[order]) and np.array_equal(c, cols[order]) and np.array_equal(v, vals[order])
    m3, n3, r, c, v = api.coo_sort_rows(M, N, rows, cols, vals, transpose=True)
    assert (m3, n3) == (N, M) and r.shape[0] == nnz and api.coo_is_row_sorted(r)


@pytest.mark.parametrize("parts", [1, 2, 3, 4, 8])
def test_partition_rows_balanced_and_order_preserving(parts):
    rng = np.random.default_rng(parts)
    M, N, K = 1000, 300, 16
    deg = (rng.pareto(1.2, M) * 3).astype(np.int64).clip(0, N)
    deg[rng.choice(M, 300, replace=False)] = 0
    rows = np.repeat(np.arange(M), deg).astype(np.int32)
    cols = np.concatenate([np.sort(rng.choice(N, d, replace=False)) for d in deg]).astype(np.int32)
    nnz = rows.shape[0]
    for align in (1, 32):
        cuts, nnz_cuts = api.partition_rows(M, rows, parts, align)
        assert cuts[0] == 0 and cuts[-1] == M and np.all(np.diff(cuts) >= 0)
        assert np.all(cuts[1:-1] % align == 0)
        assert nnz_cuts[0] == 0 and nnz_cuts[-1] == nnz
        for g in range(parts + 1):
            assert nnz_cuts[g] == np.searchsorted(rows, cuts[g], side="left")
        # each part's load is within one aligned row block of the ideal share
        worst_block = max(deg[i:i + align].sum() for i in range(0, M, align))
        for g in range(1, parts):
            assert nnz_cuts[g] >= g * nnz // parts
            assert nnz_cuts[g] - g * nnz // parts <= worst_block
    # virtual devices: shard-wise oracle results concatenate to the unsharded result
    W = rng.standard_normal((M, K)).astype(np.float32)
    H = rng.standard_normal((N, K)).astype(np.float32)
    full = oracle.cpu.sddmm_coo(rows, cols, W, H)
    cuts, nnz_cuts = api.partition_rows(M, rows, parts, 8)
    pieces = []
    for g in range(parts):
        a, b = nnz_cuts[g], nnz_cuts[g + 1]
        r0 = cuts[g]
        pieces.append(oracle.cpu.sddmm_coo(rows[a:b] - r0, cols[a:b], W[r0:cuts[g + 1]], H) if b > a else np.zeros(0, np.float32))
    assert np.array_equal(np.concatenate(pieces), full)


def test_weighted_partition_moves_cuts_towards_short_rows():
    # first half: 100 rows of 100 nonzeros; second half: 10000 rows of 1 nonzero.  Same nonzero count,
    # very different row counts: with a row cost the second block must get fewer nonzeros.
    rows = np.concatenate([np.repeat(np.arange(100), 100), 100 + np.arange(10000)]).astype(np.int32)
    M = 10100
    cuts0, nnz0 = api.partition_rows(M, rows, 2, 1)
    assert nnz0[1] == 10000 and cuts0[1] == 100
    cuts1, nnz1 = api.partition_rows(M, rows, 2, 1, row_cost=1.0)
    assert cuts1[1] > 100 and nnz1[1] > 10000
    # cost of both sides within one row of each other
    cost = lambda a, b: (b - a) + 1.0 * np.unique(rows[a:b]).size
    assert abs(cost(0, nnz1[1]) - cost(nnz1[1], rows.size)) <= 4
    for parts in (3, 8):
        c, z = api.partition_rows(M, rows, parts, 32, row_cost=2.0)
        assert c[0] == 0 and c[-1] == M and np.all(np.diff(c) >= 0) and z[-1] == rows.size


# ---- seeded synthetic matrices (sddmm_gen_open) ---------------------------------

def _is_row_sorted_unique(M, N, rows, cols):
    key = rows.astype(np.int64) * N + cols
    return bool(np.all(np.diff(key) > 0)) and rows.min() >= 0 and rows.max() < M and cols.min() >= 0 and cols.max() < N


def test_generators_have_the_benchmark_shapes():
    M, N, rows, cols, vals = api.gen_matrix("c1")
    assert (M, N, rows.size) == (4096, 4096, 16777) and _is_row_sorted_unique(M, N, rows, cols)
    assert np.all(vals == 1.0)
    M, N, rows, cols, vals = api.gen_matrix("c2")
    assert (M, N, rows.size) == (12419, 1500, 746316) and _is_row_sorted_unique(M, N, rows, cols)
    assert np.all(vals == np.round(vals)) and vals.min() >= 1 and vals.max() <= 20
    lengths = np.bincount(rows, minlength=M)
    assert lengths.max() <= N and lengths.max() > 20 * max(np.median(lengths), 1)     # heavy-tailed rows
    col_pop = np.bincount(cols, minlength=N)
    assert col_pop[:50].mean() > 5 * col_pop[-500:].mean()                          # popular columns first


def test_rmat_generator_is_skewed_and_deduplicated():
    scale, ef = 12, 8
    M, N, rows, cols, vals = api.gen_matrix(f"rmat:{scale}:{ef}")
    assert M == N == 1 << scale and _is_row_sorted_unique(M, N, rows, cols)
    assert 0.7 * ef * M < rows.size <= ef * M                                      # duplicates removed
    half = M // 2
    quad_a = np.mean((rows < half) & (cols < half))
    quad_d = np.mean((rows >= half) & (cols >= half))
    assert 0.45 < quad_a < 0.60 and 0.03 < quad_d < 0.09                           # (a, d) = (0.57, 0.05) before dedup
    assert abs(float(vals.mean())) < 0.02 and 0.97 < float(vals.std()) < 1.03      # normal(0, 1)


def test_band_generator_counts():
    M, hw, g = 700, 9, 4
    _, _, rows, cols, vals = api.gen_matrix(f"band:{M}:{hw}:{g}")
    assert _is_row_sorted_unique(M, M, rows, cols)
    lengths = np.bincount(rows, minlength=M)
    full_rows = np.nonzero(lengths == M)[0]
    col_len = np.bincount(cols, minlength=M)
    full_cols = np.nonzero(col_len == M)[0]
    assert full_rows.size == g and full_cols.size == g
    inside = np.abs(rows.astype(np.int64) - cols) <= hw
    expect_band = sum(min(M - 1, i + hw) - max(0, i - hw) + 1 for i in range(M))
    assert inside.sum() == expect_band
    outside = ~inside
    assert np.all(np.isin(rows[outside], full_rows) | np.isin(cols[outside], full_cols))


def test_generators_are_deterministic_and_seeded():
    a = api.gen_matrix("uniform:300:200:0.05")
    b = api.gen_matrix("uniform:300:200:0.05")
    c = api.gen_matrix("uniform:300:200:0.05:seed=9")
    assert a[2].size == b[2].size == c[2].size == 3000
    assert np.array_equal(a[2], b[2]) and np.array_equal(a[3], b[3])
    assert not (np.array_equal(a[2], c[2]) and np.array_equal(a[3], c[3]))
    for bad in ("nosuch:1:2", "uniform:10:10:1.5", "rmat:40:2", "band:10:1:11", "uniform:10:10:0.1:seed=x"):
        with pytest.raises(api.SddmmError):
            api.gen_matrix(bad)


# ---- formats around the loader ---------------------------------------------------

def test_symmetric_files_expand_on_request(tmp_path):
    path = tmp_path / "sym.mtx"
    path.write_text("%%MatrixMarket matrix coordinate real symmetric\n% lower triangle\n4 4 4\n1 1 2.0\n3 1 -1.5\n4 2 7\n4 4 1\n")
    M, N, rows, cols, vals = api.mtx_read(str(path))                       # as stored, like the reference
    assert (M, N, rows.size) == (4, 4, 4)
    M, N, rows, cols, vals = api.mtx_read(str(path), api.MTX_EXPAND_SYMMETRIC | api.MTX_SORT_ROWS)
    got = sorted(zip(rows.tolist(), cols.tolist(), vals.tolist()))
    assert got == [(0, 0, 2.0), (0, 2, -1.5), (1, 3, 7.0), (2, 0, -1.5), (3, 1, 7.0), (3, 3, 1.0)]
    assert api.coo_is_row_sorted(rows)
    skew = tmp_path / "skew.mtx"
    skew.write_text("%%MatrixMarket matrix coordinate integer skew-symmetric\n3 3 1\n3 1 5\n")
    _, _, rows, cols, vals = api.mtx_read(str(skew), api.MTX_EXPAND_SYMMETRIC | api.MTX_SORT_ROWS)
    assert list(zip(rows.tolist(), cols.tolist(), vals.tolist())) == [(0, 2, -5.0), (2, 0, 5.0)]
    rect = tmp_path / "rect.mtx"
    rect.write_text("%%MatrixMarket matrix coordinate real symmetric\n3 4 1\n3 1 5\n")
    with pytest.raises(api.SddmmError):
        api.mtx_read(str(rect), api.MTX_EXPAND_SYMMETRIC)


def test_docword_header_and_sorting_on_read(tmp_path):
    # headerless bag-of-words triples: documents, words, entries on three lines, then doc word count
    path = tmp_path / "docword.txt"
    path.write_text("3\n5\n4\n2 5 3\n1 2 1\n3 1 9\n1 1 4\n")
    M, N, rows, cols, vals = api.mtx_read(str(path), api.MTX_SORT_ROWS)
    assert (M, N) == (3, 5)
    assert list(zip(rows.tolist(), cols.tolist(), vals.tolist())) == [(0, 0, 4.0), (0, 1, 1.0), (1, 4, 3.0), (2, 0, 9.0)]


def test_binary_matrix_round_trip_and_corruption(tmp_path):
    M, N, rows, cols, vals = api.gen_matrix("rmat:10:6:seed=3")
    path = str(tmp_path / "m.sddmm")
    api.coo_save_binary(path, M, N, rows, cols, vals)
    M2, N2, r2, c2, v2 = api.mtx_read(path)
    assert (M2, N2) == (M, N) and np.array_equal(r2, rows) and np.array_equal(c2, cols) and np.array_equal(v2, vals)
    api.coo_save_binary(path, M, N, rows, cols, None)                       # pattern only: values read back as 1
    _, _, r3, c3, v3 = api.mtx_read(path)
    assert np.array_equal(r3, rows) and np.all(v3 == 1.0)
    api.coo_save_binary(path, M, N, rows, cols, vals)
    raw = bytearray(open(path, "rb").read())
    raw[48 + 4 * (rows.size // 2)] ^= 0x01                                   # flip one bit of a row index
    open(path, "wb").write(raw)
    with pytest.raises(api.SddmmError):
        api.mtx_read(path)
    open(path, "wb").write(raw[:100])
    with pytest.raises(api.SddmmError):
        api.mtx_read(path)


def test_c_client_of_the_abi(tmp_path):
    """A plain C99 program compiled against include/sddmm_b200.h and linked with the library."""
    import shutil
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else shutil.which("gcc")
    if cc is None:
        pytest.skip("no C compiler")
    libdir = os.path.join(root, "sddmm_gpu_b200", "csrc")
    exe = str(tmp_path / "host_only")
    build = subprocess.run([cc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(root, "include"),
                            os.path.join(root, "tests", "c_abi", "host_only.c"), "-o", exe, "-L", libdir, "-lsddmm_b200",
                            "-Wl,-rpath," + libdir], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([exe], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "FAILED" not in run.stdout


def test_shared_memory_optin_cache_is_per_device():
    """A second GPU in the same process must make its own opt-in to large dynamic shared memory."""
    assert api.lib().sddmm_selftest_optin_cache() == api.OK


def test_host_code_under_address_and_ub_sanitizers(tmp_path):
    """The host-only sources (readers, writers, converter, partitioner, generators) compiled with
    -fsanitize=address,undefined and driven through the C ABI over good, malformed and truncated inputs:
    any out-of-bounds access, leak of a closed reader or undefined arithmetic ends the run non-zero."""
    import shutil
    import subprocess
    cxx, cc = shutil.which("g++"), shutil.which("gcc")
    if not cxx or not cc:
        pytest.skip("no compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "sddmm_gpu_b200", "csrc")
    san = ["-fsanitize=address,undefined", "-fno-sanitize-recover=all", "-fno-omit-frame-pointer", "-g", "-O1"]
    objs = []
    for name in ("mtx_io.cpp", "gen.cpp"):
        o = str(tmp_path / (name + ".o"))
        r = subprocess.run([cxx, "-std=c++17", "-I", os.path.join(root, "include"), "-I", src, "-pthread", "-c",
                            os.path.join(src, name), "-o", o] + san, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        objs.append(o)
    o = str(tmp_path / "driver.o")
    r = subprocess.run([cc, "-std=c99", "-D_DEFAULT_SOURCE", "-Wall", "-I", os.path.join(root, "include"), "-c",
                        os.path.join(root, "tests", "c_abi", "host_sanitize.c"), "-o", o] + san, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    exe = str(tmp_path / "host_sanitize")
    r = subprocess.run([cxx, o] + objs + ["-o", exe, "-pthread"] + san, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    work = tmp_path / "files"
    work.mkdir()
    run = subprocess.run([exe, str(work)], capture_output=True, text=True,
                         env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1"))
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-3000:]
    assert "FAILED" not in run.stdout and run.stdout.count("ok:") >= 40
