"""CPU tests of the preprocessing restatement (oracle/preprocess_oracle.py):
vectorised form vs the literal per-window transcription, the invariants that follow from
the reference's kernels (src/utils.cu), and the golden arrays dumped from the rebuilt
reference extension on a B200 (tests/golden/tcb_ref_*.npz)."""
import numpy as np
import pytest

from conftest import GOLDEN, random_csr
from oracle import preprocess_oracle as po

ARRAYS = ["rowWindowOffset", "sortedRowWindows", "tcblock_rowid", "tcblocktile_id", "tcblock_offset",
          "sparseAToXidx", "tcbBitMap", "blockPartition", "edgeToColumn", "edgeToRow"]


def popcount64(x):
    x = x.astype(np.uint64)
    return np.array([bin(int(v)).count("1") for v in x], dtype=np.int64)


def check_invariants(rowptr, colidx, n, bw, t, unique_cols_per_row=True):
    nrw = (n + 15) // 16
    rwo = t["rowWindowOffset"].astype(np.int64)
    assert rwo[0] == 0 and np.all(np.diff(rwo) >= 0) and rwo[-1] == t["nTCB"]
    off = t["tcblock_offset"].astype(np.int64)
    assert off[0] == 0 and off[-1] == len(colidx) and np.all(np.diff(off) >= 0)
    # edges of a window == edges of its TCBs (reference check: scripts/graph_stat/paper_graph_stat.py:69-72)
    for w in range(nrw):
        e = int(rowptr[min(16 * w + 16, n)]) - int(rowptr[16 * w])
        assert off[rwo[w + 1]] - off[rwo[w]] == e
    wpt = 16 * bw // 64
    if unique_cols_per_row:
        pc = popcount64(t["tcbBitMap"]).reshape(-1, wpt).sum(1) if t["nTCB"] else np.zeros(0, np.int64)
        assert np.array_equal(pc, np.diff(off))
    # column list: ascending inside a window over the occupied slots, zero padding
    atox = t["sparseAToXidx"]
    e2c = t["edgeToColumn"].astype(np.int64)
    deg = np.diff(rowptr.astype(np.int64))
    win = np.repeat(np.arange(n), deg) // 16
    assert np.array_equal(atox[rwo[win] * bw + e2c], colidx)
    srt = t["sortedRowWindows"]
    assert sorted(srt.tolist()) == list(range(nrw))
    cnt = np.diff(rwo)[srt]
    assert np.all(np.diff(cnt) <= 0)
    ties = np.diff(cnt) == 0
    assert np.all(np.diff(srt.astype(np.int64))[ties] > 0)


@pytest.mark.parametrize("n,deg,seed,sort_cols,dups", [
    (1, 1, 0, True, False), (15, 3, 1, True, False), (16, 3, 2, True, False), (17, 5, 3, True, False),
    (100, 7, 4, True, False), (130, 20, 5, False, False), (97, 9, 6, False, True), (64, 40, 7, True, False),
])
@pytest.mark.parametrize("bw", [8, 16])
def test_vectorised_matches_literal(n, deg, seed, sort_cols, dups, bw):
    rowptr, colidx = random_csr(n, deg, seed, sort_cols, dups)
    a = po.preprocess(colidx, rowptr, n, 16, bw)
    b = po.preprocess_loops(colidx, rowptr, n, 16, bw)
    assert a["nTCB"] == b["nTCB"]
    for k in ARRAYS:
        assert a[k].dtype == b[k].dtype, k
        assert np.array_equal(a[k], b[k]), k
    check_invariants(rowptr, colidx, n, bw, a, unique_cols_per_row=not dups)


def test_exact_multiple_of_block_width():
    # a window with exactly 2*bw distinct columns must give 2 TCBs, not 3 (src/utils.cu:148)
    n = 32
    cols = np.arange(32, dtype=np.int32)
    rowptr = np.zeros(n + 1, np.int32)
    rowptr[1:] = 32  # row 0 holds all 32 columns, the other rows are empty
    t = po.preprocess(cols, rowptr, n, 16, 16)
    assert t["blockPartition"].tolist() == [2, 0]
    assert t["nTCB"] == 2
    assert t["sortedRowWindows"].tolist() == [0, 1]


def test_empty_graph_and_empty_windows():
    n = 40
    rowptr = np.zeros(n + 1, np.int32)
    t = po.preprocess(np.zeros(0, np.int32), rowptr, n)
    assert t["nTCB"] == 0 and t["rowWindowOffset"].tolist() == [0, 0, 0, 0]
    assert t["tcblock_offset"].tolist() == [0]
    assert t["sortedRowWindows"].tolist() == [0, 1, 2]
    # caller-provided blockPartition is left alone for windows without edges (src/utils.cu:141-142)
    t = po.preprocess(np.zeros(0, np.int32), rowptr, n, block_partition_init=np.array([5, 0, 1], np.int32))
    assert t["blockPartition"].tolist() == [5, 0, 1]


def test_bitmap_layout_matches_kernel_reads():
    # the fused kernel reads word t*4 + (warp%2)*2 + i/2 and bit 63 - 2*lane - i%2
    # (src/F3S_kernel.cu:1663-1667): lane = 4*(row%8) + (col%8)/2, warp%2 = col/8, i/2 = row/8
    n = 16
    for r in (0, 5, 8, 15):
        for c in (0, 7, 8, 13):
            cols = np.arange(16, dtype=np.int32)
            rowptr = np.zeros(n + 1, np.int32)
            # row r has the single column c; one extra row holds all 16 columns so that rank == column
            other = (r + 1) % 16
            deg = np.zeros(n, np.int64)
            deg[r] = 1
            deg[other] = 16
            rowptr[1:] = np.cumsum(deg)
            colidx = np.zeros(17, np.int32)
            colidx[rowptr[r]] = c
            colidx[rowptr[other]:rowptr[other] + 16] = cols
            t = po.preprocess(colidx, rowptr, n, 16, 16)
            word = (c // 8) * 2 + r // 8
            lane, i = 4 * (r % 8) + (c % 8) // 2, 2 * (r // 8) + (c % 2)
            bit = 63 - 2 * lane - i % 2
            assert (int(t["tcbBitMap"][word]) >> bit) & 1


def test_edge_to_row_defect_emulation():
    # src/utils.cu:348: with N > 1024 the grid is wider than 32 and a row longer than 32 edges
    # is only partly written; below that the defect is inert.
    n = 2048
    deg = np.ones(n, np.int64)
    deg[100] = 200
    rowptr = np.zeros(n + 1, np.int32)
    rowptr[1:] = np.cumsum(deg)
    rng = np.random.default_rng(0)
    colidx = np.concatenate([np.sort(rng.choice(n, size=d, replace=False)) for d in deg]).astype(np.int32)
    good = po.preprocess(colidx, rowptr, n)
    bad = po.preprocess(colidx, rowptr, n, emulate_edge_to_row_defect=True)
    grid = 64
    o = np.arange(200)
    expect = np.where(o % grid < 32, 100, 0)
    assert np.array_equal(bad["edgeToRow"][rowptr[100]:rowptr[101]], expect)
    for k in ("rowWindowOffset", "sortedRowWindows", "tcblock_rowid", "tcblock_offset", "sparseAToXidx",
              "blockPartition", "edgeToColumn"):
        assert np.array_equal(good[k], bad[k]), k
    assert not np.array_equal(good["tcbBitMap"], bad["tcbBitMap"])
    small = po.preprocess(colidx[: rowptr[1000]], rowptr[:1001], 1000, emulate_edge_to_row_defect=True)
    assert np.array_equal(small["edgeToRow"], po.preprocess(colidx[: rowptr[1000]], rowptr[:1001], 1000)["edgeToRow"])


GOLDEN_TCB = sorted(GOLDEN.glob("tcb_ref_*.npz"))


@pytest.mark.parametrize("path", GOLDEN_TCB, ids=[p.stem for p in GOLDEN_TCB])
def test_against_reference_arrays(path):
    """Arrays dumped from the rebuilt reference extension running on a B200."""
    g = np.load(path)
    bw = int(g["block_w"])
    n = int(g["num_nodes"])
    defect = bool(g["unmodified_reference"])
    t = po.preprocess(g["colidx"], g["rowptr"], n, 16, bw, emulate_edge_to_row_defect=defect)
    assert t["nTCB"] == int(g["nTCB"])
    for k in ARRAYS:
        assert np.array_equal(t[k], g[k]), f"{path.name}: {k}"


def test_golden_reference_arrays_present():
    assert GOLDEN_TCB, "tests/golden/tcb_ref_*.npz missing: the preprocessing oracle would be unpinned"


def _byte_perm(a, b, sel):
    """PTX prmt.b32 (default mode): result byte i = byte (sel >> 4i) & 7 of the pair {b, a} (a = bytes 0..3)."""
    by = [(a >> (8 * i)) & 255 for i in range(4)] + [(b >> (8 * i)) & 255 for i in range(4)]
    return sum(by[(sel >> (4 * i)) & 7] << (8 * i) for i in range(4))


def _tile_ids_from_words(words, bw):
    """Host model of the fill kernel's sort-free path (fused3s_b200/csrc/preprocess.cu, tile_bytes_of_block):
    the occupancy words of one TC block regrouped into 32-bit row-major words, tile id = 32 * word + clz."""
    if bw == 16:
        m = []
        for h in range(2):
            lh, ll = words[h] >> 32, words[h] & 0xFFFFFFFF
            rh, rl = words[2 + h] >> 32, words[2 + h] & 0xFFFFFFFF
            m += [_byte_perm(lh, rh, 0x3726), _byte_perm(lh, rh, 0x1504),
                  _byte_perm(ll, rl, 0x3726), _byte_perm(ll, rl, 0x1504)]
    else:
        m = [x for h in range(2) for x in (words[h] >> 32, words[h] & 0xFFFFFFFF)]
    out = []
    for k, x in enumerate(m):
        while x:
            z = 32 - x.bit_length()
            out.append(32 * k + z)
            x &= ~(0x80000000 >> z)
    return out


@pytest.mark.parametrize("bw", [16, 8])
def test_tile_ids_follow_from_occupancy_words_when_rows_ascend(bw):
    """What the CUDA fill kernel relies on for sorted CSR rows: inside a TC block the CSR order of the edges is
    the row-major order of its occupancy bits, so tcblocktile_id and tcblock_offset are functions of tcbBitMap
    (src/utils.cu:173-224 writes them edge by edge).  Checked on the oracle's arrays, which are pinned to the
    reference's."""
    rowptr, colidx = random_csr(700, 60, 17, sort_cols=True, duplicates=False)
    t = po.preprocess(colidx, rowptr, 700, 16, bw)
    wpt = 16 * bw // 64
    bm = t["tcbBitMap"].astype(np.uint64).reshape(-1, wpt)
    off = t["tcblock_offset"]
    assert t["nTCB"] > 100
    for b in range(t["nTCB"]):
        ids = _tile_ids_from_words([int(w) for w in bm[b]], bw)
        assert len(ids) == off[b + 1] - off[b]
        assert ids == [int(x) for x in t["tcblocktile_id"][off[b]:off[b + 1]]], b
    # with an unsorted row the property fails, which is why the kernel checks the order first
    rowptr2, colidx2 = random_csr(64, 40, 18, sort_cols=False, duplicates=False)
    t2 = po.preprocess(colidx2, rowptr2, 64, 16, bw)
    bm2 = t2["tcbBitMap"].astype(np.uint64).reshape(-1, wpt)
    off2 = t2["tcblock_offset"]
    same = all(_tile_ids_from_words([int(w) for w in bm2[b]], bw)
               == [int(x) for x in t2["tcblocktile_id"][off2[b]:off2[b + 1]]] for b in range(t2["nTCB"]))
    assert not same
