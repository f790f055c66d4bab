// Block plan: layout of the plan buffer and the Philox4x32-10 draw shared by host and device.
#pragma once
#include <stdint.h>

#include "../../include/sparsedrop.h"

#if defined(__CUDACC__)
#define SD_HD __host__ __device__
#else
#define SD_HD
#endif

namespace sd {

constexpr int kPlanHeaderInts = 16;
enum PlanHeader { H_NNZ = 0, H_SDD_ITEMS = 1, H_NDROP = 2, H_R = 3, H_C = 4, H_MAX_ROW = 5, H_MAX_COL = 6 };

SD_HD inline int64_t plan_align16(int64_t x) { return (x + 15) & ~int64_t(15); }

// Byte offsets of every array of the plan buffer for an R x C grid of 128x128 tiles.
SD_HD inline sd_plan_layout plan_layout(int R, int C) {
    sd_plan_layout L;
    const int64_t RC = int64_t(R) * C;
    int64_t off = 0;
    L.header = off;     off = plan_align16(off + 4 * kPlanHeaderInts);
    L.row_ptr = off;    off = plan_align16(off + 4 * (int64_t(R) + 1));
    L.col_idx = off;    off = plan_align16(off + 4 * RC);
    L.col_ptr = off;    off = plan_align16(off + 4 * (int64_t(C) + 1));
    L.row_idx = off;    off = plan_align16(off + 4 * RC);
    L.kept_pairs = off; off = plan_align16(off + 8 * RC);
    L.drop_pairs = off; off = plan_align16(off + 8 * RC);
    L.row_order = off;  off = plan_align16(off + 4 * int64_t(R));
    L.col_order = off;  off = plan_align16(off + 4 * int64_t(C));
    L.sdd_items = off;  off = plan_align16(off + 12 * int64_t(R) * ((C + 1) / 2));
    L.mask = off;       off = plan_align16(off + RC);
    L.total_bytes = off;
    return L;
}

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11).
// Returns the first output word for counter (c0, c1, c2, c3) and key (k0, k1).
SD_HD inline uint32_t philox4x32_10_x(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                      uint32_t k1) {
    for (int round = 0; round < 10; ++round) {
        const uint64_t p0 = uint64_t(0xD2511F53u) * c0;
        const uint64_t p1 = uint64_t(0xCD9E8D57u) * c2;
        const uint32_t n0 = uint32_t(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n1 = uint32_t(p1);
        const uint32_t n2 = uint32_t(p0 >> 32) ^ c3 ^ k1;
        const uint32_t n3 = uint32_t(p0);
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c0;
}

// Drop decision of logical block `index` for (seed, offset): u in [0,1) with 24 bits, dropped iff u < p.
SD_HD inline bool philox_drop(uint64_t seed, uint64_t offset, uint64_t index, float p) {
    const uint32_t x = philox4x32_10_x(uint32_t(index), uint32_t(index >> 32), uint32_t(offset),
                                       uint32_t(offset >> 32), uint32_t(seed), uint32_t(seed >> 32));
    const float u = float(x >> 8) * (1.0f / 16777216.0f);
    return u < p;
}

}  // namespace sd
