// CPU check of the slice planner of the host-streamed step (nabla_b200/csrc/host_plan.h).
//
// The per-chunk ownership below is written chunk by chunk the way the kernels derive it
// (head elements with chunk 0, 4-element items per chunk, tail elements with the final
// chunk; rows without an aligned body are cut at plain 4096-element boundaries).  The
// planner's closed-form ranges must equal the union of those sets for every chunk range,
// and a plan must cover every row exactly once, in order, in slices of the asked length.
#include <stdio.h>
#include <stdlib.h>

#include <random>
#include <vector>

#include "../nabla_b200/csrc/host_plan.h"

using namespace nbo;

static int g_fail = 0;
#define CHECK(c, ...)                                              \
    do {                                                           \
        if (!(c)) {                                                \
            if (g_fail++ < 10) { printf("FAIL %s:%d ", __FILE__, __LINE__); printf(__VA_ARGS__); printf("\n"); } \
        }                                                          \
    } while (0)

// marks owner[e] = c for every element chunk c owns
static void mark_chunk(std::vector<int64_t> &owner, uint64_t n, uint32_t head, uint64_t c)
{
    auto own = [&](uint64_t lo, uint64_t hi) {
        for (uint64_t e = lo; e < hi; ++e) {
            CHECK(owner[e] < 0, "element %llu owned twice (n=%llu head=%u)", (unsigned long long)e, (unsigned long long)n, head);
            owner[e] = (int64_t)c;
        }
    };
    if (head == 0xffffffffu) {
        uint64_t b = c * kChunkElems, e = b + kChunkElems < n ? b + kChunkElems : n;
        own(b, e);
        return;
    }
    uint64_t hd = head < n ? head : n;
    uint64_t body_items = (n - hd) >> 2;
    uint64_t i0 = c * kChunkItems;
    uint64_t i1 = i0 + kChunkItems < body_items ? i0 + kChunkItems : body_items;
    if (i0 > body_items) i0 = body_items;
    if (i1 > i0) own(hd + (i0 << 2), hd + (i1 << 2));
    if (c == 0) own(0, hd);
    bool last = (c + 1) * kChunkElems >= n;
    if (last) own(hd + (body_items << 2), n);
}

static void check_row(uint64_t n, uint32_t head, std::mt19937_64 &rng)
{
    uint64_t nc = row_chunks(n);
    std::vector<int64_t> owner(n, -1);
    for (uint64_t c = 0; c < nc; ++c) mark_chunk(owner, n, head, c);
    for (uint64_t e = 0; e < n; ++e) CHECK(owner[e] >= 0, "element %llu unowned (n=%llu head=%u)", (unsigned long long)e, (unsigned long long)n, head);
    for (int t = 0; t < 24; ++t) {
        uint64_t a = nc ? rng() % (nc + 1) : 0, b = nc ? rng() % (nc + 1) : 0;
        if (t == 0) { a = 0; b = nc; }
        if (a > b) std::swap(a, b);
        ElemRange r = chunk_range_elems(n, head, a, b);
        CHECK(r.lo <= r.hi && r.hi <= n, "range order n=%llu head=%u a=%llu b=%llu", (unsigned long long)n, head, (unsigned long long)a, (unsigned long long)b);
        for (uint64_t e = 0; e < n; ++e) {
            bool in = e >= r.lo && e < r.hi;
            bool want = owner[e] >= (int64_t)a && owner[e] < (int64_t)b;
            if (in != want) {
                CHECK(false, "n=%llu head=%u chunks [%llu,%llu): element %llu in=%d want=%d (range %llu..%llu)",
                      (unsigned long long)n, head, (unsigned long long)a, (unsigned long long)b, (unsigned long long)e,
                      (int)in, (int)want, (unsigned long long)r.lo, (unsigned long long)r.hi);
                break;
            }
        }
    }
}

static void check_plan(const std::vector<uint64_t> &row_n, const std::vector<uint32_t> &row_head,
                       const std::vector<int32_t> &row_group, int32_t ngroups, uint64_t slice_chunks)
{
    HostPlan plan = plan_host_slices(row_n, row_head, row_group, ngroups, slice_chunks);
    // the chunk list as the library builds it: group-major, rows in table order
    std::vector<uint32_t> group_begin(ngroups + 1, 0);
    uint64_t pos = 0;
    for (int32_t g = 0; g < ngroups; ++g) {
        group_begin[g] = (uint32_t)pos;
        for (size_t r = 0; r < row_n.size(); ++r)
            if (row_group[r] == g) pos += row_chunks(row_n[r]);
    }
    group_begin[ngroups] = (uint32_t)pos;
    std::vector<uint64_t> next_elem(row_n.size(), 0);
    uint32_t expect_chunk = 0;
    int32_t g = 0;
    for (const Slice &s : plan.slices) {
        while (g < ngroups && group_begin[g + 1] == group_begin[g]) ++g;            // empty groups
        while (g < ngroups && expect_chunk == group_begin[g + 1]) { ++g; while (g < ngroups && group_begin[g + 1] == group_begin[g]) ++g; }
        CHECK(s.group == g, "slice group %d, expected %d", s.group, g);
        CHECK(s.chunk_begin == expect_chunk, "slice begins at %u, expected %u", s.chunk_begin, expect_chunk);
        CHECK(s.chunk_end > s.chunk_begin && s.chunk_end - s.chunk_begin <= slice_chunks, "slice length");
        CHECK(s.chunk_end <= group_begin[s.group + 1], "slice crosses its group");
        expect_chunk = s.chunk_end;
        uint64_t chunks_in_copies = 0;
        for (uint32_t k = s.copy_begin; k < s.copy_end; ++k) {
            const SliceCopy &c = plan.copies[k];
            CHECK(row_group[c.row] == s.group, "copy row in another group");
            CHECK(c.lo == next_elem[c.row], "row %u: copy starts at %llu, expected %llu", c.row, (unsigned long long)c.lo, (unsigned long long)next_elem[c.row]);
            CHECK(c.hi > c.lo && c.hi <= row_n[c.row], "copy range");
            next_elem[c.row] = c.hi;
            (void)chunks_in_copies;
        }
    }
    CHECK(expect_chunk == pos, "plan covers %u of %llu chunks", expect_chunk, (unsigned long long)pos);
    for (size_t r = 0; r < row_n.size(); ++r)
        CHECK(next_elem[r] == row_n[r], "row %zu covered to %llu of %llu", r, (unsigned long long)next_elem[r], (unsigned long long)row_n[r]);
}

// Sharded plans: every rank's slices together must copy every element of the bucket exactly once, each slice's
// ranges must lie inside the rank's shard, and all ranks must be able to agree on the number of slices.
static void check_sharded(const std::vector<uint64_t> &numel, const std::vector<int32_t> &group_of, int32_t ngroups,
                          int world, uint64_t slice_chunks)
{
    uint64_t total = 0;
    for (uint64_t n : numel) total += n;
    uint64_t shard = (total + world - 1) / world;
    shard = (shard + 7) & ~7ull;
    if (shard == 0) shard = 8;
    std::vector<int> covered(total, 0);
    for (int q = 0; q < world; ++q) {
        std::vector<ShardRow> rows = shard_rows(numel, group_of, q, shard);
        std::vector<uint64_t> row_n;
        std::vector<uint32_t> row_head;
        std::vector<int32_t> row_group;
        uint64_t owned = 0;
        for (const ShardRow &r : rows) {
            CHECK(r.bucket_off >= (uint64_t)q * shard && r.bucket_off + r.n <= (uint64_t)(q + 1) * shard, "row outside its shard");
            row_n.push_back(r.n); row_head.push_back(bucket_row_head(r.bucket_off)); row_group.push_back(r.group);
            owned += r.n;
        }
        uint64_t want = total > (uint64_t)q * shard ? total - (uint64_t)q * shard : 0;
        if (want > shard) want = shard;
        CHECK(owned == want, "rank %d owns %llu of %llu elements", q, (unsigned long long)owned, (unsigned long long)want);
        check_plan(row_n, row_head, row_group, ngroups, slice_chunks);
        HostPlan plan = plan_host_slices(row_n, row_head, row_group, ngroups, slice_chunks);
        for (const SliceCopy &c : plan.copies)
            for (uint64_t e = rows[c.row].bucket_off + c.lo; e < rows[c.row].bucket_off + c.hi; ++e) covered[e] += 1;
    }
    for (uint64_t e = 0; e < total; ++e)
        if (covered[e] != 1) { CHECK(false, "bucket element %llu copied %d times (world %d)", (unsigned long long)e, covered[e], world); break; }
}

int main()
{
    std::mt19937_64 rng(1234);
    const uint64_t sizes[] = {0, 1, 2, 3, 4, 5, 7, 8, 4092, 4093, 4094, 4095, 4096, 4097, 4098, 4099, 4100, 4101, 4103,
                              8191, 8192, 8193, 8195, 8199, 12288, 12289, 12291, 12295, 20000, 40961, 65536 + 5};
    const uint32_t heads[] = {0, 1, 2, 3, 0xffffffffu};
    for (uint64_t n : sizes)
        for (uint32_t h : heads) check_row(n, h, rng);
    for (int t = 0; t < 300; ++t) check_row(rng() % 70000, heads[rng() % 5], rng);

    for (int t = 0; t < 400; ++t) {
        int rows = 1 + (int)(rng() % 12);
        int32_t ngroups = 1 + (int32_t)(rng() % 3);
        std::vector<uint64_t> n(rows);
        std::vector<uint32_t> hd(rows);
        std::vector<int32_t> gr(rows);
        for (int r = 0; r < rows; ++r) {
            n[r] = (rng() % 5 == 0) ? rng() % 6 : rng() % 60000;
            hd[r] = heads[rng() % 5];
            gr[r] = (int32_t)(rng() % ngroups);
        }
        uint64_t slice_chunks = 1 + rng() % 9;
        if (t % 7 == 0) slice_chunks = 1u << 20;
        check_plan(n, hd, gr, ngroups, slice_chunks);
    }
    for (int t = 0; t < 200; ++t) {
        int tensors = 1 + (int)(rng() % 10);
        int32_t ngroups = 1 + (int32_t)(rng() % 3);
        std::vector<uint64_t> n(tensors);
        std::vector<int32_t> gr(tensors);
        for (int r = 0; r < tensors; ++r) {
            n[r] = (rng() % 5 == 0) ? rng() % 6 : rng() % 50000;
            gr[r] = (int32_t)(rng() % ngroups);
        }
        const int worlds[] = {1, 2, 3, 4, 8};
        check_sharded(n, gr, ngroups, worlds[rng() % 5], 1 + rng() % 6);
    }
    if (g_fail) { printf("HOST_PLAN_FAILED %d\n", g_fail); return 1; }
    printf("HOST_PLAN_OK\n");
    return 0;
}
