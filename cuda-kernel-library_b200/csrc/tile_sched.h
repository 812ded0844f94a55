// Tile schedule of the tensor-core GEMM, as pure integer functions shared by
// the host planner, the kernels and the fix-up pass (so all three agree by
// construction) and unit-testable on a CPU.
//
// A GEMM is cut into tiles_m x tiles_n output tiles, each accumulated over
// k_blocks pipeline steps.  `units` schedulable workers (one CTA, or one CTA
// pair for the 2-CTA kernel) run persistently:
//
//   * stream-K region (run first): the last sk_tiles tiles are laid end to end
//     as sk_tiles * k_blocks iterations and cut into `units` equal contiguous
//     ranges.  A unit whose range covers a whole tile writes C directly; a
//     range that starts or stops inside a tile yields a PARTIAL accumulator.
//     The partials of a split tile are added in ascending unit order
//     (deterministic) either by the unit that holds the tile's first k blocks
//     (fused: the others park their partials in FP32 workspace slots and raise
//     a flag) or by a separate fix-up pass over parked partials of all holders;
//   * data-parallel region (run after): tiles [0, dp_tiles) are dealt
//     round-robin; unit u computes tiles u, u + units, ... whole.
//
// The reference has no counterpart: it launches one CTA per tile and leaves
// the last wave under-filled (src/gemm/gemm_mma_opt.cu:223-225).
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define CKL_HD __host__ __device__ __forceinline__
#else
#define CKL_HD inline
#endif

namespace ckl {

struct Schedule {
    int tiles_m;
    int tiles_n;
    int k_blocks;
    int units;
    int dp_tiles;
    int sk_tiles;
    int group_m;  // tile rows per raster group (L2 reuse of B columns / A rows)
    long long sk_iters;
};

struct Segment {
    int tile;      // linear tile index in raster order
    int kb_begin;  // first k block
    int kb_end;    // one past the last k block
    int slot;      // workspace slot for a partial, -1 when the unit owns the whole tile
};

// Raster order: groups of `group_m` tile rows; inside a group the row index
// runs fastest, so the tiles in flight at one time form a compact block of
// the output and share A row panels and B column panels in L2.
CKL_HD void tile_coords(const Schedule& s, int tile, int* tm, int* tn) {
    const int per_group = s.group_m * s.tiles_n;
    const int group = tile / per_group;
    const int first_m = group * s.group_m;
    int rows = s.tiles_m - first_m;
    if (rows > s.group_m) {
        rows = s.group_m;
    }
    const int in_group = tile - group * per_group;
    *tm = first_m + in_group % rows;
    *tn = in_group / rows;
}

CKL_HD long long sk_range_begin(const Schedule& s, int u) {
    return s.sk_iters * static_cast<long long>(u) / s.units;
}

// Cursor over the segments of one unit, in execution order.
struct SegmentCursor {
    int unit;
    int dp_next;        // next data-parallel tile, or >= dp_tiles when done
    long long sk_cur;   // next stream-K iteration
    long long sk_end;
};

CKL_HD SegmentCursor make_cursor(const Schedule& s, int u) {
    SegmentCursor c;
    c.unit = u;
    c.dp_next = u;
    c.sk_cur = sk_range_begin(s, u);
    c.sk_end = sk_range_begin(s, u + 1);
    return c;
}

// The stream-K range comes FIRST, the unit's whole tiles after it: a unit that has to wait
// for other units' partials and add them (fused fix-up) does so while its MMA warp is already
// busy with the whole tiles, and the launch ends with an ordinary tile, not with a reduction.
CKL_HD bool next_segment(const Schedule& s, SegmentCursor* c, Segment* out) {
    if (c->sk_cur < c->sk_end) {
        const long long t = c->sk_cur / s.k_blocks;
        const int kb0 = static_cast<int>(c->sk_cur - t * s.k_blocks);
        long long stop = (t + 1) * s.k_blocks;
        if (stop > c->sk_end) {
            stop = c->sk_end;
        }
        const int kb1 = static_cast<int>(stop - t * s.k_blocks);
        out->tile = s.dp_tiles + static_cast<int>(t);
        out->kb_begin = kb0;
        out->kb_end = kb1;
        if (kb0 == 0 && kb1 == s.k_blocks) {
            out->slot = -1;
        } else {
            // A range can enter a tile mid-way only with its first segment and
            // leave one mid-way only with its last: two slots per unit suffice.
            out->slot = 2 * c->unit + (kb0 == 0 ? 1 : 0);
        }
        c->sk_cur = stop;
        return true;
    }
    if (c->dp_next < s.dp_tiles) {
        out->tile = c->dp_next;
        out->kb_begin = 0;
        out->kb_end = s.k_blocks;
        out->slot = -1;
        c->dp_next += s.units;
        return true;
    }
    return false;
}

// First unit whose stream-K range contains iteration `it`.
CKL_HD int sk_owner_of(const Schedule& s, long long it) {
    int u = static_cast<int>(it * s.units / (s.sk_iters > 0 ? s.sk_iters : 1));
    if (u >= s.units) {
        u = s.units - 1;
    }
    while (u > 0 && sk_range_begin(s, u) > it) {
        --u;
    }
    while (u + 1 < s.units && sk_range_begin(s, u + 1) <= it) {
        ++u;
    }
    return u;
}

constexpr int kMaxFixupSlots = 512;

// The workspace slots holding the partial accumulators of split tile
// `sk_tile`, in the (ascending unit) order the fix-up pass adds them.
// Returns 0 when a single unit owned the whole tile and wrote C itself.
CKL_HD int fixup_slots(const Schedule& s, int sk_tile, int* slots, int max_slots) {
    const long long it0 = static_cast<long long>(sk_tile) * s.k_blocks;
    const long long it1 = it0 + s.k_blocks;
    int count = 0;
    for (int u = sk_owner_of(s, it0); u < s.units; ++u) {
        const long long b = sk_range_begin(s, u);
        const long long e = sk_range_begin(s, u + 1);
        if (b >= it1) {
            break;
        }
        if (e <= it0 || e <= b) {
            continue;
        }
        const long long lo = b > it0 ? b : it0;
        const long long hi = e < it1 ? e : it1;
        if (lo == it0 && hi == it1) {
            return 0;
        }
        if (count < max_slots) {
            slots[count] = 2 * u + (lo == it0 ? 1 : 0);
        }
        ++count;
    }
    return count < max_slots ? count : max_slots;
}

}  // namespace ckl
