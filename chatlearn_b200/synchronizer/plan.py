"""Trainer → rollout weight reshard planner.

The reference plans this with ``ShardedTensorInfo`` algebra, per-engine mappers
and a bucketising planner (chatlearn/synchronizer/mappers/*.py,
chatlearn/synchronizer/planners/*.py, chatlearn/utils/mappings/sharded_tensor_info.py)
and executes it as pack → NCCL all-to-all → CUDA-IPC → unpack+cast
(chatlearn/synchronizer/comm.py:92-286).  Here both sides publish their leaves as
rectangles of the canonical HuggingFace tensors (``models.nn.layout``); the plan
is the intersection of source and destination rectangles, emitted as flat copy
descriptors

    (src rank, src buffer, src offset, src row stride,
     dst buffer, dst offset, dst row stride, rows, cols)

that a single kernel executes by *pulling* from peer memory over NVLink with the
dtype cast fused in (``ops.native`` ``weight_sync``), or that the portable
executor runs with point-to-point messages.  QKV packing, gate/up packing, GQA
KV-head replication, TP re-splitting and EP expert re-homing need no special
cases: they are all "this rectangle goes there".
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from chatlearn_b200.models.nn.layout import Leaf

Rect = Tuple[int, int, int, int]  # row0, col0, rows, cols


@dataclass
class BufferInfo:
    """One flat buffer (a parameter block) of one rank.

    ``shard``: ``None`` when the rank holds the whole buffer; else ``(lo, hi)``
    element range it owns (ZeRO-style even sharding of the flat block)."""
    name: str
    numel: int
    dtype: str
    shard: Optional[Tuple[int, int]] = None


@dataclass
class LeafPlacement:
    leaf: Leaf
    buffer: str                 # BufferInfo.name
    offset: int                 # element offset of the leaf inside the buffer


@dataclass
class RankLayout:
    """Everything one rank publishes to the planner (pure metadata, picklable)."""
    rank: int
    buffers: Dict[str, BufferInfo] = field(default_factory=dict)
    leaves: List[LeafPlacement] = field(default_factory=list)


@dataclass(frozen=True)
class CopyDesc:
    src_rank: int
    src_buffer: str
    src_offset: int
    src_stride: int
    dst_rank: int
    dst_buffer: str
    dst_offset: int
    dst_stride: int
    rows: int
    cols: int
    hf_name: str = ""

    @property
    def numel(self):
        return self.rows * self.cols


def _intersect(a: Rect, b: Rect) -> Optional[Rect]:
    r0, c0 = max(a[0], b[0]), max(a[1], b[1])
    r1, c1 = min(a[0] + a[2], b[0] + b[2]), min(a[1] + a[3], b[1] + b[3])
    if r1 <= r0 or c1 <= c0:
        return None
    return (r0, c0, r1 - r0, c1 - c0)


def _subtract(a: Rect, b: Rect) -> List[Rect]:
    """``a`` minus ``b`` (``b`` inside ``a``) as up to four rectangles."""
    out = []
    ar1, ac1 = a[0] + a[2], a[1] + a[3]
    br1, bc1 = b[0] + b[2], b[1] + b[3]
    if b[0] > a[0]:
        out.append((a[0], a[1], b[0] - a[0], a[3]))
    if br1 < ar1:
        out.append((br1, a[1], ar1 - br1, a[3]))
    if b[1] > a[1]:
        out.append((b[0], a[1], b[2], b[1] - a[1]))
    if bc1 < ac1:
        out.append((b[0], bc1, b[2], ac1 - bc1))
    return out


@dataclass
class _SrcPiece:
    rank: int
    buffer: str
    shard: Optional[Tuple[int, int]]
    rect: Rect                  # in HF coordinates
    base: int                   # element offset (in the full buffer) of HF (rect.row0, rect.col0)
    stride: int                 # elements between consecutive rows in the buffer


def _leaf_pieces(layout: RankLayout) -> Dict[str, List[_SrcPiece]]:
    out: Dict[str, List[_SrcPiece]] = {}
    for lp in layout.leaves:
        lf = lp.leaf
        rows, cols = lf.matrix_shape
        slab = rows * cols
        buf = layout.buffers[lp.buffer]
        for s in lf.segments:
            base = lp.offset + s.dst_index * slab + s.dst_start[0] * cols + s.dst_start[1]
            out.setdefault(s.hf_name, []).append(_SrcPiece(
                layout.rank, lp.buffer, buf.shard,
                (s.src_start[0], s.src_start[1], s.extent[0], s.extent[1]), base, cols))
    return out


def _split_by_shard(base: int, stride: int, rows: int, cols: int, lo: int, hi: int):
    """Parts of the strided 2-D region ``{base + r*stride + c}`` that fall in the
    element range ``[lo, hi)``, as ``(row0, col0, rows, cols)`` sub-regions: the
    rows wholly inside the range form one 2-D part; the (at most two) rows that
    straddle ``lo`` or ``hi`` contribute 1-row parts."""
    if rows <= 0 or cols <= 0 or hi <= lo:
        return
    stride = max(stride, 1)
    ra = max(-(-(lo - base) // stride), 0)                 # first row starting at or after lo
    rb = min((hi - cols - base) // stride + 1, rows)       # one past the last row ending by hi
    full0, full1 = min(ra, rows), max(rb, 0)
    if full1 > full0:
        yield (full0, 0, full1 - full0, cols)
    else:
        full0 = full1 = -1
    for r in sorted({ra - 1, rb}):
        if r < 0 or r >= rows or (full0 <= r < full1):
            continue
        start = base + r * stride
        s, e = max(start, lo), min(start + cols, hi)
        if e > s:
            yield (r, s - start, 1, e - s)


def build_plan(src_layouts: List[RankLayout], dst_layouts: List[RankLayout],
               prefer_local: bool = True) -> Dict[int, List[CopyDesc]]:
    """Copy descriptors per destination rank.

    Sources that hold identical data (data-parallel replicas, or the shards of a
    ZeRO-sharded buffer) are chosen so that (1) a rank copies from itself when it
    can and (2) the remaining traffic is spread over the sender ranks evenly
    (largest-first greedy, the role of the reference's sender-group balancing in
    chatlearn/synchronizer/planners/base_planner.py:167-192)."""
    src_index: Dict[str, List[_SrcPiece]] = {}
    for lay in src_layouts:
        for name, pieces in _leaf_pieces(lay).items():
            src_index.setdefault(name, []).extend(pieces)
    sent: Dict[int, int] = {lay.rank: 0 for lay in src_layouts}
    plan: Dict[int, List[CopyDesc]] = {}
    for dlay in dst_layouts:
        descs: List[CopyDesc] = []
        for lp in dlay.leaves:
            lf = lp.leaf
            rows, cols = lf.matrix_shape
            slab = rows * cols
            for s in lf.segments:
                cands = src_index.get(s.hf_name)
                if not cands:
                    raise KeyError(f"no source holds '{s.hf_name}' needed by rank {dlay.rank}")
                want: List[Rect] = [(s.src_start[0], s.src_start[1], s.extent[0], s.extent[1])]
                dst_base = lp.offset + s.dst_index * slab + s.dst_start[0] * cols + s.dst_start[1]

                def emit(piece: _SrcPiece, inter: Rect, lo_hi):
                    # region of the source buffer that holds `inter`
                    sb = piece.base + (inter[0] - piece.rect[0]) * piece.stride + (inter[1] - piece.rect[1])
                    db = dst_base + (inter[0] - s.src_start[0]) * cols + (inter[1] - s.src_start[1])
                    if lo_hi is None:
                        parts = [(0, 0, inter[2], inter[3])]
                        shard_lo = 0
                    else:
                        parts = list(_split_by_shard(sb, piece.stride, inter[2], inter[3], *lo_hi))
                        shard_lo = lo_hi[0]
                    got = []
                    for (r0, c0, nr, nc) in parts:
                        descs.append(CopyDesc(piece.rank, piece.buffer,
                                              sb + r0 * piece.stride + c0 - shard_lo, piece.stride,
                                              dlay.rank, lp.buffer, db + r0 * cols + c0, cols,
                                              nr, nc, s.hf_name))
                        sent[piece.rank] = sent.get(piece.rank, 0) + nr * nc
                        got.append((inter[0] + r0, inter[1] + c0, nr, nc))
                    return got

                # order candidates: local first, then least-loaded sender
                def order_key(p: _SrcPiece):
                    local = 0 if (prefer_local and p.rank == dlay.rank) else 1
                    return (local, sent.get(p.rank, 0), p.rank)

                progress = True
                while want and progress:
                    progress = False
                    for piece in sorted(cands, key=order_key):
                        new_want: List[Rect] = []
                        for w in want:
                            inter = _intersect(w, piece.rect)
                            if inter is None:
                                new_want.append(w)
                                continue
                            got = emit(piece, inter, piece.shard)
                            rem = [w]
                            for g in got:
                                nxt = []
                                for rr in rem:
                                    ii = _intersect(rr, g)
                                    if ii is None:
                                        nxt.append(rr)
                                    else:
                                        nxt.extend(_subtract(rr, ii))
                                rem = nxt
                            if got:
                                progress = True
                            new_want.extend(rem)
                        want = new_want
                        if not want:
                            break
                if want:
                    raise ValueError(f"'{s.hf_name}' region {want[:2]} needed by rank {dlay.rank} "
                                     f"is not covered by any source shard")
        plan[dlay.rank] = descs
    return plan


def validate_plan(plan: Dict[int, List[CopyDesc]], dst_layouts: List[RankLayout]):
    """Every destination leaf element must be written exactly once."""
    for dlay in dst_layouts:
        need = sum(s.extent[0] * s.extent[1] for lp in dlay.leaves for s in lp.leaf.segments)
        have = sum(d.numel for d in plan[dlay.rank])
        if need != have:
            raise ValueError(f"rank {dlay.rank}: plan writes {have} elements, layout has {need}")
        # no overlapping writes
        by_buf: Dict[str, List[Tuple[int, int]]] = {}
        for d in plan[dlay.rank]:
            if d.cols == d.dst_stride or d.rows == 1:
                by_buf.setdefault(d.dst_buffer, []).append((d.dst_offset, d.dst_offset + d.rows * d.cols
                                                            if d.cols == d.dst_stride else d.dst_offset + d.cols))
        for buf, spans in by_buf.items():
            spans.sort()
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                if b0 < a1:
                    raise ValueError(f"rank {dlay.rank}: overlapping writes in {buf}")


def plan_stats(plan: Dict[int, List[CopyDesc]], elem_bytes: int = 2) -> Dict[str, float]:
    local = remote = n = 0
    per_sender: Dict[int, int] = {}
    for dst, descs in plan.items():
        for d in descs:
            n += 1
            if d.src_rank == dst:
                local += d.numel
            else:
                remote += d.numel
                per_sender[d.src_rank] = per_sender.get(d.src_rank, 0) + d.numel
    return {"descriptors": n, "local_bytes": local * elem_bytes, "remote_bytes": remote * elem_bytes,
            "max_sender_bytes": max(per_sender.values(), default=0) * elem_bytes}


# ---------------------------------------------------------------------------- memory-budgeted iterations
def split_rows(d: CopyDesc, max_elems: int) -> List[CopyDesc]:
    """Cut a rectangle into row bands of at most ``max_elems`` elements (a single row is never cut)."""
    if d.numel <= max_elems or d.rows <= 1:
        return [d]
    band = max(1, max_elems // max(d.cols, 1))
    out = []
    for r0 in range(0, d.rows, band):
        n = min(band, d.rows - r0)
        out.append(CopyDesc(d.src_rank, d.src_buffer, d.src_offset + r0 * d.src_stride, d.src_stride,
                            d.dst_rank, d.dst_buffer, d.dst_offset + r0 * d.dst_stride, d.dst_stride, n, d.cols, d.hf_name))
    return out


def build_iterations(plan: Dict[int, List[CopyDesc]], elem_size: int, bucket_bytes: int,
                     budget_bytes: Optional[Dict[int, int]] = None) -> List[Dict[Tuple[int, int], List[CopyDesc]]]:
    """Schedule the remote pieces of a plan into iterations with bounded staging memory.

    Parity: chatlearn/synchronizer/planners/tensor_planner.py:39-176 (``_check_constraint`` / ``build_iteration``:
    a bucket per sender and receiver group never exceeds ``bucket_size``, and the buckets a GPU holds in one
    iteration, sent and received, fit into ``max_memory_fraction`` of its memory).  The point-to-point executor
    packs what one rank sends another into one message, so per iteration a rank stages the messages it sends and
    the messages it receives.  Here: every message is at most ``bucket_bytes``; the bytes a rank stages in one
    iteration (both directions) are at most ``budget_bytes[rank]`` (no entry: unbounded); pieces larger than a
    bucket are cut into row bands first.  Pieces are placed first-fit in a canonical order, so every rank derives
    the same schedule from the same plan.  Returns, per iteration, ``{(src, dst): [pieces]}``; pieces whose source
    is their destination are not scheduled (they are local copies).
    """
    budget_bytes = budget_bytes or {}
    max_elems = max(1, bucket_bytes // elem_size)
    pieces: List[CopyDesc] = []
    for dst in sorted(plan):
        for d in plan[dst]:
            if d.src_rank != dst:
                pieces.extend(split_rows(d, max_elems))
    pieces.sort(key=lambda d: (d.src_rank, d.dst_rank))          # stable: plan order within a pair
    iters: List[Dict[Tuple[int, int], List[CopyDesc]]] = []
    staged: List[Dict[int, int]] = []                              # per iteration: bytes staged per rank
    msg: List[Dict[Tuple[int, int], int]] = []                     # per iteration: bytes per message
    for d in pieces:
        nb = d.numel * elem_size
        pair = (d.src_rank, d.dst_rank)
        for need in (d.src_rank, d.dst_rank):
            if need in budget_bytes and nb > budget_bytes[need]:
                raise RuntimeError(f"parameter sync: a piece of {nb} bytes ({d.hf_name or d.src_buffer}) does not fit "
                                   f"the staging budget of rank {need} ({budget_bytes[need]} bytes); lower the bucket size")
        placed = False
        for it in range(len(iters)):
            if msg[it].get(pair, 0) + nb > bucket_bytes and msg[it].get(pair, 0) > 0:
                continue
            if any(staged[it].get(r, 0) + nb > budget_bytes[r] for r in pair if r in budget_bytes):
                continue
            placed = True
            break
        if not placed:
            iters.append({}); staged.append({}); msg.append({})
            it = len(iters) - 1
        iters[it].setdefault(pair, []).append(d)
        msg[it][pair] = msg[it].get(pair, 0) + nb
        for r in pair:
            staged[it][r] = staged[it].get(r, 0) + nb
    return iters


def iteration_stats(iters, elem_size: int) -> Dict[str, float]:
    peak = 0
    for it in iters:
        per_rank: Dict[int, int] = {}
        for (s, d), ds in it.items():
            nb = sum(x.numel for x in ds) * elem_size
            per_rank[s] = per_rank.get(s, 0) + nb
            per_rank[d] = per_rank.get(d, 0) + nb
        peak = max([peak] + list(per_rank.values()))
    return {"iterations": len(iters), "peak_staged_mb": round(peak / 2 ** 20, 2)}
