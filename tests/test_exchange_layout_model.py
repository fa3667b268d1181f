"""A host-side model of the two-shot exchange's index arithmetic (kernels.cuh: two_shot_step and the
chunk loop of ar_body), checked for shapes no GPU test covers: every staging vector a rank polls
is written exactly once by the peer it expects, the gather area is covered exactly, the CTAs of a
cluster partition their row and their share of the slice, the chunks partition the rows, and all
offsets stay inside the workspace regions the host code sizes (core.cu: gpuk_ws_create).
The model uses the planner of the library for tile, cluster, chunk and grid, so it also pins the
contract between the planner and the kernels.
"""
import itertools

import pytest

from gpuk_b200 import cabi

RS_SLACK_VECS = (1 << 20) // 16      # kRsSlack: room for ceil(row_vecs / N) rounding in the scatter slots


def _model(world, tokens, hidden, resident_ctas):
    p = cabi.plan(world, tokens * hidden, hidden, oneshot_max_bytes=1)      # force the two-shot exchange
    assert not p.one_shot
    rows, rv, cl, R = p.rows, p.row_vecs, p.cluster, p.rows_per_chunk
    vpr = -(-rv // world)
    seg = -(-rv // cl)
    nchunks = -(-rows // R)
    clusters = max(1, min(p.grid, resident_ctas) // cl)
    clusters = min(clusters, nchunks)
    nb = clusters * cl
    B, VPT = p.threads, p.vpt
    ibb = -(-VPT // world)
    sub = -(-vpr // cl)
    cap_vecs = -(-(tokens * hidden * 2) // (256 * world)) * 256 * world // 16
    slot_vecs = cap_vecs // world + RS_SLACK_VECS
    scatter_written = {}      # (dest, src, index) -> count
    gather_written = {}       # (dest, vector) -> count
    scatter_read = set()
    gather_read = set()
    rows_done = [0] * rows
    for rank in range(world):
        for vb in range(nb):
            cid, cr = vb // cl, vb % cl
            nk = (nchunks - cid + clusters - 1) // clusters if cid < nchunks else 0
            for k in range(nk):
                r0 = (cid + k * clusters) * R
                r1 = min(r0 + R, rows)
                for row in range(r0, r1):
                    if rank == 0 and cr == 0:
                        rows_done[row] += 1
                    v0 = cr * seg
                    end = min(v0 + seg, rv)
                    # scatter and finish: thread t, slot i -> vector v0 + t + i * B
                    covered = [v0 + t + i * B for i in range(VPT) for t in range(B) if v0 + t + i * B < end]
                    assert sorted(covered) == list(range(v0, max(v0, end))), (row, cr)
                    for v in covered:
                        owner = v // vpr
                        if owner != rank:
                            idx = row * vpr + (v - owner * vpr)
                            assert idx < slot_vecs
                            scatter_written[(owner, rank, idx)] = scatter_written.get((owner, rank, idx), 0) + 1
                        gather_read.add((rank, row * rv + v))
                        assert row * rv + v < cap_vecs
                    # slice reduction: thread t, slot b -> slice vector vl0 + t + b * B
                    vl0, vl1 = cr * sub, min(cr * sub + sub, vpr)
                    mine = [vl0 + t + b * B for b in range(ibb) for t in range(B) if vl0 + t + b * B < vl1]
                    assert sorted(mine) == list(range(vl0, max(vl0, vl1))), (row, cr, "slice share")
                    for vl in mine:
                        if rank * vpr + vl < rv:
                            for src in range(world):
                                if src != rank:
                                    scatter_read.add((rank, src, row * vpr + vl))
                            for dest in range(world):
                                key = (dest, row * rv + rank * vpr + vl)
                                gather_written[key] = gather_written.get(key, 0) + 1
    assert rows_done == [1] * rows
    assert all(c == 1 for c in scatter_written.values()) and all(c == 1 for c in gather_written.values())
    assert set(scatter_written) == scatter_read
    assert set(gather_written) == gather_read
    return p


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("tokens,hidden", [(1, 8192), (3, 2056), (5, 136), (9, 7168), (37, 1024), (33, 4104), (70, 8), (12, 16384)])
def test_two_shot_indices_cover_staging_exactly_once(world, tokens, hidden):
    for resident in (296, 64, 8):       # all chunks resident, a few chunks per cluster, many chunks per cluster
        _model(world, tokens, hidden, resident)


def test_model_sees_clusters_and_multi_row_chunks():
    assert _model(8, 8, 8192, 296).cluster == 8
    assert _model(2, 64, 8192, 296).cluster > 1
    # more rows than resident CTAs: several rows per chunk, the last chunk ragged
    for world, tokens, hidden in ((8, 2001, 64), (2, 1501, 1024), (4, 1203, 520)):
        p = _model(world, tokens, hidden, 296)
        assert p.rows_per_chunk > 1 and p.cluster == 1 and tokens % p.rows_per_chunk
    big = cabi.plan(8, 16384 * 7168, 7168, oneshot_max_bytes=1)
    assert big.rows_per_chunk > 1 and big.cluster == 1
