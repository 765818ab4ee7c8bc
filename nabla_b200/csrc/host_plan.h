// Slice planner of the host-streamed step (nbo_step_mixed_host / nbo_zero1_step_host).
//
// Pure host arithmetic, no CUDA: the step cuts the chunk list into slices, and for every
// slice it must copy exactly the elements the update kernel touches for that chunk range:
// gradients host -> device before the launch, parameters device -> host after it.  The
// geometry restated here is the one chunk_view() in kernels.cuh gives the kernels:
//
//   row without an aligned body (head == 0xffffffff): chunk c owns [c*4096, min(n, (c+1)*4096))
//   aligned row with `head` leading elements:         chunk c owns the 4-element items
//       [head + c*4096, min(head + (c+1)*4096, head + 4*body_items)), chunk 0 also owns the
//       head [0, head) and the final chunk also owns the tail [head + 4*body_items, n).
//
// so consecutive chunk ranges of one row own consecutive, disjoint element ranges.
#pragma once
#include <stdint.h>

#include <vector>

#include "types.h"

namespace nbo {

struct ElemRange {
    uint64_t lo, hi;  // elements [lo, hi) of the row
};

inline uint64_t row_chunks(uint64_t n) { return (n + kChunkElems - 1) / kChunkElems; }

// Elements of a row of `n` elements owned by its chunks [a, b), 0 <= a <= b <= row_chunks(n).
inline ElemRange chunk_range_elems(uint64_t n, uint32_t head, uint64_t a, uint64_t b)
{
    const uint64_t nc = row_chunks(n);
    ElemRange r;
    if (a >= b) { r.lo = r.hi = 0; return r; }
    if (head == 0xffffffffu) {
        r.lo = a * kChunkElems;
        r.hi = b * kChunkElems < n ? b * kChunkElems : n;
        return r;
    }
    const uint64_t hd = head < n ? head : n;
    const uint64_t body_end = hd + (((n - hd) >> 2) << 2);  // first tail element
    uint64_t lo = hd + a * kChunkElems, hi = hd + b * kChunkElems;
    if (lo > body_end) lo = body_end;
    if (hi > body_end) hi = body_end;
    r.lo = a == 0 ? 0 : lo;
    r.hi = b == nc ? n : hi;
    return r;
}

// One copy of the plan: elements [lo, hi) of table row `row`.
struct SliceCopy {
    uint32_t row;
    uint64_t lo, hi;
};

// One slice: chunk-list entries [chunk_begin, chunk_end) of one group and the rows they touch.
struct Slice {
    int32_t group;
    uint32_t chunk_begin, chunk_end;
    uint32_t copy_begin, copy_end;  // range in HostPlan::copies
};

struct HostPlan {
    std::vector<Slice> slices;
    std::vector<SliceCopy> copies;
};

// One table row of a ZeRO-1 rank: the part of tensor `tensor` that falls into the rank's shard.
struct ShardRow {
    uint64_t tensor;      // index in the declared list
    uint64_t offset;      // first element of the piece inside its tensor
    uint64_t n;           // elements
    uint64_t bucket_off;  // element offset in the flat bucket
    int32_t group;
};

// The rows of rank `rank` for a flat bucket holding the tensors in list order, every rank owning `shard`
// consecutive elements.  Every rank can derive every other rank's rows (and from them its slice plan):
// the result depends on the declared sizes alone.
inline std::vector<ShardRow> shard_rows(const std::vector<uint64_t> &numel, const std::vector<int32_t> &group_of,
                                        int rank, uint64_t shard)
{
    std::vector<ShardRow> out;
    const uint64_t begin = (uint64_t)rank * shard, end = begin + shard;
    uint64_t off = 0;
    for (size_t t = 0; t < numel.size(); ++t) {
        uint64_t lo = off > begin ? off : begin;
        uint64_t hi = off + numel[t] < end ? off + numel[t] : end;
        if (hi > lo) out.push_back(ShardRow{(uint64_t)t, lo - off, hi - lo, lo, group_of[t]});
        off += numel[t];
    }
    return out;
}

// Leading elements of a bucket row that precede the next 4-element boundary of the bucket.
inline uint32_t bucket_row_head(uint64_t bucket_off) { return (uint32_t)((4 - (bucket_off & 3)) & 3); }

// Rows are given in chunk-list order: the list holds group 0's rows first (each row's chunks
// consecutive, rows in table order), then group 1's, and so on.  `row_n`, `row_head`,
// `row_group` are indexed by table row; `slice_chunks` >= 1 is the slice length in chunks.
inline HostPlan plan_host_slices(const std::vector<uint64_t> &row_n, const std::vector<uint32_t> &row_head,
                                 const std::vector<int32_t> &row_group, int32_t ngroups, uint64_t slice_chunks)
{
    HostPlan plan;
    if (slice_chunks == 0) slice_chunks = 1;
    uint64_t list_pos = 0;  // chunk-list index of the next row's first chunk
    for (int32_t g = 0; g < ngroups; ++g) {
        Slice cur{g, (uint32_t)list_pos, (uint32_t)list_pos, (uint32_t)plan.copies.size(), (uint32_t)plan.copies.size()};
        auto flush = [&]() {
            cur.copy_end = (uint32_t)plan.copies.size();
            if (cur.chunk_end > cur.chunk_begin) plan.slices.push_back(cur);
            cur.chunk_begin = cur.chunk_end;
            cur.copy_begin = cur.copy_end;
        };
        for (size_t row = 0; row < row_n.size(); ++row) {
            if (row_group[row] != g) continue;
            const uint64_t nc = row_chunks(row_n[row]);
            uint64_t a = 0;
            while (a < nc) {
                uint64_t room = slice_chunks - (cur.chunk_end - cur.chunk_begin);
                uint64_t b = a + room < nc ? a + room : nc;
                ElemRange r = chunk_range_elems(row_n[row], row_head[row], a, b);
                if (r.hi > r.lo) plan.copies.push_back(SliceCopy{(uint32_t)row, r.lo, r.hi});
                cur.chunk_end += (uint32_t)(b - a);
                a = b;
                if (cur.chunk_end - cur.chunk_begin == slice_chunks) flush();
            }
            list_pos += nc;
        }
        flush();
    }
    return plan;
}

}  // namespace nbo
