// Block-plan kernel: draws (or reads) the drop mask of an R x C grid of 128x128 tiles and
// compacts it, in one launch (one CTA; a cluster of eight for grids of thousands of tiles), into every index list the GEMM kernels walk
// (CSR, CSC, kept/dropped pair lists, heaviest-first orders, paired SDD work items).
//
// Replaces, device-side and without any host synchronisation:
//   blockwise_dropout_mask        flash_dropout/functional/utils.py:11-16
//   mask_to_increment_table       flash_dropout/functional/utils.py:19-69   (CSR form)
//   torch.nonzero(~mask)          flash_dropout/functional/blockwise_dropout_matmul_triton.py:48
//   mask.T                        flash_dropout/functional/blockwise_dropout_matmul_cuda.py:50 (CSC form)
//
// The work is a few KB of integer traffic: the launch is latency-bound, not HBM-bound.
#include <cooperative_groups.h>

#include <cstdlib>

#include "sd_common.h"
#include "sd_plan.cuh"
#include "sd_ptx.cuh"

namespace cg = cooperative_groups;

namespace sd {

constexpr int kPlanThreads = 1024;
constexpr int kSmemMaskBytes = 32768;

// Exclusive scan of one value per thread over the whole CTA (kPlanThreads threads).
// `total` receives the sum.  warp_sums is 32 ints of shared memory.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
    }
    __syncthreads();   // protects warp_sums against a previous call's readers
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = warp_sums[lane];
        int wi = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int n = __shfl_up_sync(0xffffffffu, wi, d);
            if (lane >= d) wi += n;
        }
        warp_sums[lane] = wi - w;   // exclusive warp offsets
        if (lane == 31) warp_sums[32] = wi;
    }
    __syncthreads();
    total = warp_sums[32];
    return warp_sums[warp] + incl - v;
}

// The same for two values per thread in one pass (three barriers instead of six): both sums must stay below 2^31.
// pair_sums is 33 64-bit words of shared memory.
__device__ __forceinline__ void block_exclusive_scan_pair(int a, int b, unsigned long long* pair_sums, int& off_a,
                                                          int& off_b, int& total_a, int& total_b) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned long long v = (unsigned long long)(unsigned)a | ((unsigned long long)(unsigned)b << 32);
    unsigned long long incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned long long n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
    }
    __syncthreads();   // protects pair_sums against a previous call's readers
    if (lane == 31) pair_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const unsigned long long w = pair_sums[lane];
        unsigned long long wi = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned long long n = __shfl_up_sync(0xffffffffu, wi, d);
            if (lane >= d) wi += n;
        }
        pair_sums[lane] = wi - w;   // exclusive warp offsets
        if (lane == 31) pair_sums[32] = wi;
    }
    __syncthreads();
    const unsigned long long tot = pair_sums[32], mine = pair_sums[warp] + incl - v;
    total_a = int(unsigned(tot));
    total_b = int(unsigned(tot >> 32));
    off_a = int(unsigned(mine));
    off_b = int(unsigned(mine >> 32));
}

struct PlanArgs {
    unsigned char* plan;
    int R, C, rep, rep_c;   // logical block = rep x rep_c tiles (rows x columns)
    int from_seed;
    unsigned long long seed, offset;
    unsigned long long* counter;   // optional device counter added to `offset`, incremented by this launch
    float p;
    const unsigned char* mask_in;
    long long mask_rs, mask_cs;
    unsigned char* mask_out;
    // one launch for several plans (plan_bits_batch_kernel): the CTAs share `counter`; plan j of n draws with
    // offset + j + *counter, and the last CTA to arrive (counted in *batch_arrivals) advances the counter by n
    unsigned int* batch_arrivals;
    int batch_n;
};

__global__ void __launch_bounds__(kPlanThreads, 1) plan_kernel(PlanArgs a) {
    __shared__ unsigned char smask[kSmemMaskBytes];
    __shared__ int warp_sums[33];
    __shared__ int bins[kPlanThreads];
    __shared__ int s_max_row, s_max_col;

    const int R = a.R, C = a.C, rep = a.rep, rep_c = a.rep_c;
    const int RC = R * C;
    const int Cm = (C + rep_c - 1) / rep_c;
    const sd_plan_layout L = plan_layout(R, C);
    int* header = reinterpret_cast<int*>(a.plan + L.header);
    int* row_ptr = reinterpret_cast<int*>(a.plan + L.row_ptr);
    int* col_idx = reinterpret_cast<int*>(a.plan + L.col_idx);
    int* col_ptr = reinterpret_cast<int*>(a.plan + L.col_ptr);
    int* row_idx = reinterpret_cast<int*>(a.plan + L.row_idx);
    int* kept_pairs = reinterpret_cast<int*>(a.plan + L.kept_pairs);
    int* drop_pairs = reinterpret_cast<int*>(a.plan + L.drop_pairs);
    int* row_order = reinterpret_cast<int*>(a.plan + L.row_order);
    int* col_order = reinterpret_cast<int*>(a.plan + L.col_order);
    int* sdd_items = reinterpret_cast<int*>(a.plan + L.sdd_items);
    unsigned char* gmask = a.plan + L.mask;
    const bool in_smem = RC <= kSmemMaskBytes;
    unsigned char* m = in_smem ? smask : gmask;

    if (threadIdx.x == 0) { s_max_row = 0; s_max_col = 0; }
    grid_dep_launch();
    grid_dep_wait();   // the counter, a caller's mask and the plan buffer may belong to the previous kernel
    const unsigned long long offset = a.offset + (a.counter ? *a.counter : 0ull);

    // ---- phase 0: the drop decision of every tile (1 = dropped)
    for (int i = threadIdx.x; i < RC; i += kPlanThreads) {
        const int r = i / C, c = i - r * C;
        const int lr = r / rep, lc = c / rep_c;
        bool drop;
        if (a.from_seed) {
            drop = philox_drop(a.seed, offset, (unsigned long long)lr * Cm + lc, a.p);
            if (a.mask_out && r == lr * rep && c == lc * rep_c) a.mask_out[(long long)lr * Cm + lc] = drop;
        } else {
            drop = a.mask_in[lr * a.mask_rs + lc * a.mask_cs] != 0;
        }
        gmask[i] = drop;
        if (in_smem) smask[i] = drop;
    }
    __syncthreads();

    // ---- phase 1: rows.  Thread t owns rows [t*rpt, (t+1)*rpt).
    {
        const int rpt = (R + kPlanThreads - 1) / kPlanThreads;
        const int r0 = min(R, int(threadIdx.x) * rpt), r1 = min(R, r0 + rpt);
        int kept = 0, items = 0, mx = 0;
        for (int r = r0; r < r1; ++r) {
            int cnt = 0;
            for (int c = 0; c < C; ++c) cnt += (m[r * C + c] == 0);
            kept += cnt;
            items += (cnt + 1) >> 1;
            mx = max(mx, cnt);
        }
        int nnz, n_items, dummy;
        int kept_off = block_exclusive_scan(kept, warp_sums, nnz);
        int item_off = block_exclusive_scan(items, warp_sums, n_items);
        (void)dummy;
        if (mx) atomicMax(&s_max_row, mx);
        for (int r = r0; r < r1; ++r) {
            row_ptr[r] = kept_off;
            int drop_off = r * C - kept_off;   // dropped tiles before row r
            int first = -1;
            for (int c = 0; c < C; ++c) {
                if (m[r * C + c] == 0) {
                    col_idx[kept_off] = c;
                    kept_pairs[2 * kept_off] = r;
                    kept_pairs[2 * kept_off + 1] = c;
                    ++kept_off;
                    if (first < 0) {
                        first = c;
                    } else {
                        sdd_items[3 * item_off] = r;
                        sdd_items[3 * item_off + 1] = first;
                        sdd_items[3 * item_off + 2] = c;
                        ++item_off;
                        first = -1;
                    }
                } else {
                    drop_pairs[2 * drop_off] = r;
                    drop_pairs[2 * drop_off + 1] = c;
                    ++drop_off;
                }
            }
            if (first >= 0) {
                sdd_items[3 * item_off] = r;
                sdd_items[3 * item_off + 1] = first;
                sdd_items[3 * item_off + 2] = -1;
                ++item_off;
            }
        }
        if (threadIdx.x == 0) {
            row_ptr[R] = nnz;
            header[H_NNZ] = nnz;
            header[H_SDD_ITEMS] = n_items;
            header[H_NDROP] = RC - nnz;
            header[H_R] = R;
            header[H_C] = C;
        }
    }

    // ---- phase 2: columns.
    if (R <= 4 * C) {
        // wide or square grid: thread t owns columns [t*cpt, (t+1)*cpt) and walks their rows
        const int cpt = (C + kPlanThreads - 1) / kPlanThreads;
        const int c0 = min(C, int(threadIdx.x) * cpt), c1 = min(C, c0 + cpt);
        int kept = 0, mx = 0;
        for (int c = c0; c < c1; ++c) {
            int cnt = 0;
            for (int r = 0; r < R; ++r) cnt += (m[r * C + c] == 0);
            kept += cnt;
            mx = max(mx, cnt);
        }
        int nnz;
        int off = block_exclusive_scan(kept, warp_sums, nnz);
        if (mx) atomicMax(&s_max_col, mx);
        for (int c = c0; c < c1; ++c) {
            col_ptr[c] = off;
            for (int r = 0; r < R; ++r)
                if (m[r * C + c] == 0) row_idx[off++] = r;
        }
        if (threadIdx.x == 0) col_ptr[C] = nnz;
    } else {
        // tall grid (e.g. the im2col matrix of a conv: thousands of row blocks, a handful of K tiles):
        // one column at a time, every thread counts its own chunk of rows, a CTA-wide scan orders them
        const int rpt = (R + kPlanThreads - 1) / kPlanThreads;
        const int r0 = min(R, int(threadIdx.x) * rpt), r1 = min(R, r0 + rpt);
        int col_start = 0;
        for (int c = 0; c < C; ++c) {
            int cnt = 0;
            for (int r = r0; r < r1; ++r) cnt += (m[r * C + c] == 0);
            int col_total;
            int off = col_start + block_exclusive_scan(cnt, warp_sums, col_total);
            for (int r = r0; r < r1; ++r)
                if (m[r * C + c] == 0) row_idx[off++] = r;
            if (threadIdx.x == 0) {
                col_ptr[c] = col_start;
                if (col_total > s_max_col) s_max_col = col_total;
            }
            col_start += col_total;
        }
        if (threadIdx.x == 0) col_ptr[C] = col_start;
    }
    __syncthreads();   // row_ptr / col_ptr visible to the whole CTA

    // ---- phase 3: heaviest-first orders (a scheduling hint: any permutation is valid).
    //   n <= 1024 : stable rank sort, exact and deterministic
    //   n  > 1024 : counting sort; keys are exact while the largest count fits the 1024 bins,
    //               otherwise scaled (monotone, so the order is still non-increasing per bin)
    for (int pass = 0; pass < 2; ++pass) {
        const int n = pass == 0 ? R : C;
        const int full = pass == 0 ? C : R;   // largest possible count
        const int* ptr = pass == 0 ? row_ptr : col_ptr;
        int* order = pass == 0 ? row_order : col_order;
        if (n <= kPlanThreads) {
            if (int(threadIdx.x) < n) bins[threadIdx.x] = ptr[threadIdx.x + 1] - ptr[threadIdx.x];
            __syncthreads();
            if (int(threadIdx.x) < n) {
                const int mine = bins[threadIdx.x];
                int rank = 0;
                for (int j = 0; j < n; ++j) {
                    const int other = bins[j];
                    rank += (other > mine) || (other == mine && j < int(threadIdx.x));
                }
                order[rank] = threadIdx.x;
            }
            __syncthreads();
            continue;
        }
        auto key_of = [&](int i) {
            const int k = full - (ptr[i + 1] - ptr[i]);
            return full < kPlanThreads ? k : int((long long)k * (kPlanThreads - 1) / full);
        };
        bins[threadIdx.x] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += kPlanThreads) atomicAdd(&bins[key_of(i)], 1);
        __syncthreads();
        int total;
        const int mine = bins[threadIdx.x];
        const int start = block_exclusive_scan(mine, warp_sums, total);
        bins[threadIdx.x] = start;
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += kPlanThreads) order[atomicAdd(&bins[key_of(i)], 1)] = i;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        header[H_MAX_ROW] = s_max_row;
        header[H_MAX_COL] = s_max_col;
        if (a.counter) *a.counter = offset - a.offset + 1;   // every thread read it before the first barrier
    }
}

// Fast path for grids with at most 32 K tiles per row (K <= 4096) and at most kBitsMaxRows row blocks: a row of
// the mask is one 32-bit word (bit c set = tile (r, c) kept), produced by a warp ballot, and every list position is
// a popcount of that word, so all lists are written in parallel, a warp per row.  Same outputs as plan_kernel.
constexpr int kBitsMaxRows = 3072;


__device__ __forceinline__ void plan_bits_body(const PlanArgs& a) {
    __shared__ unsigned keepmask[kBitsMaxRows];
    __shared__ int s_row_ptr[kBitsMaxRows];
    __shared__ int s_item_ptr[kBitsMaxRows];
    __shared__ unsigned long long pair_sums[33];
    __shared__ int col_chunk[32][33];
    __shared__ int s_col_total[32];
    __shared__ int s_col_ptr[33];
    __shared__ int bins[40];
    __shared__ int s_max_row;

    const int R = a.R, C = a.C, rep = a.rep, rep_c = a.rep_c;
    const int Cm = (C + rep_c - 1) / rep_c;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const sd_plan_layout L = plan_layout(R, C);
    int* header = reinterpret_cast<int*>(a.plan + L.header);
    int* row_ptr = reinterpret_cast<int*>(a.plan + L.row_ptr);
    int* col_idx = reinterpret_cast<int*>(a.plan + L.col_idx);
    int* col_ptr = reinterpret_cast<int*>(a.plan + L.col_ptr);
    int* row_idx = reinterpret_cast<int*>(a.plan + L.row_idx);
    int* kept_pairs = reinterpret_cast<int*>(a.plan + L.kept_pairs);
    int* drop_pairs = reinterpret_cast<int*>(a.plan + L.drop_pairs);
    int* row_order = reinterpret_cast<int*>(a.plan + L.row_order);
    int* col_order = reinterpret_cast<int*>(a.plan + L.col_order);
    int* sdd_items = reinterpret_cast<int*>(a.plan + L.sdd_items);
    unsigned char* gmask = a.plan + L.mask;
    grid_dep_launch();
    grid_dep_wait();   // the counter, a caller's mask and the plan buffer may belong to the previous kernel
    const unsigned long long offset = a.offset + (a.counter ? *a.counter : 0ull);
    if (threadIdx.x == 0) s_max_row = 0;
    if (threadIdx.x < 40) bins[threadIdx.x] = 0;

    // ---- the drop decisions, one tile per thread; kept tiles set their bit in the row word
    for (int r = threadIdx.x; r < R; r += kPlanThreads) keepmask[r] = 0u;
    __syncthreads();
    for (int i = threadIdx.x; i < R * C; i += kPlanThreads) {
        const int r = i / C, c = i - r * C;
        const int lr = r / rep, lc = c / rep_c;
        bool drop;
        if (a.from_seed) {
            drop = philox_drop(a.seed, offset, (unsigned long long)lr * Cm + lc, a.p);
            if (a.mask_out && r == lr * rep && c == lc * rep_c) a.mask_out[(long long)lr * Cm + lc] = drop;
        } else {
            drop = a.mask_in[lr * a.mask_rs + lc * a.mask_cs] != 0;
        }
        gmask[i] = drop;
        if (!drop) atomicOr(&keepmask[r], 1u << c);
    }
    __syncthreads();

    // ---- row offsets: thread t owns rows [t*rpt, (t+1)*rpt)
    int nnz, n_items;
    {
        const int rpt = (R + kPlanThreads - 1) / kPlanThreads;
        const int r0 = min(R, int(threadIdx.x) * rpt), r1 = min(R, r0 + rpt);
        int kept = 0, items = 0, mx = 0;
        for (int r = r0; r < r1; ++r) {
            const int cnt = __popc(keepmask[r]);
            kept += cnt;
            items += (cnt + 1) >> 1;
            mx = max(mx, cnt);
        }
        int kept_off, item_off;
        block_exclusive_scan_pair(kept, items, pair_sums, kept_off, item_off, nnz, n_items);
        if (mx) atomicMax(&s_max_row, mx);
        for (int r = r0; r < r1; ++r) {
            const int cnt = __popc(keepmask[r]);
            s_row_ptr[r] = kept_off;
            s_item_ptr[r] = item_off;
            row_ptr[r] = kept_off;
            kept_off += cnt;
            item_off += (cnt + 1) >> 1;
        }
        if (threadIdx.x == 0) row_ptr[R] = nnz;
    }
    __syncthreads();

    // ---- row lists, one tile per thread: positions are popcounts of the row word below this column
    for (int i = threadIdx.x; i < R * C; i += kPlanThreads) {
        const int r = i / C, c = i - r * C;
        const unsigned mask = keepmask[r];
        const int base = s_row_ptr[r];
        const int j = __popc(mask & ((1u << c) - 1u));           // kept tiles left of this column
        if ((mask >> c) & 1u) {
            col_idx[base + j] = c;
            kept_pairs[2 * (base + j)] = r;
            kept_pairs[2 * (base + j) + 1] = c;
            if ((j & 1) == 0) {                                  // first tile of a pair: its partner is the next kept column
                const unsigned above = c == 31 ? 0u : mask & ~((2u << c) - 1u);
                int* it = sdd_items + 3 * (s_item_ptr[r] + (j >> 1));
                it[0] = r;
                it[1] = c;
                it[2] = above ? __ffs(above) - 1 : -1;
            }
        } else {
            const int d = r * C - base + (c - j);                // dropped tiles before this one
            drop_pairs[2 * d] = r;
            drop_pairs[2 * d + 1] = c;
        }
    }

    // ---- columns: warp w owns the row chunk [w*rpw, (w+1)*rpw); lane = column
    const int rpw = (R + 31) / 32;
    const int cr0 = min(R, warp * rpw), cr1 = min(R, cr0 + rpw);
    {
        int cnt = 0;
        for (int r = cr0; r < cr1; ++r) cnt += (keepmask[r] >> lane) & 1u;
        col_chunk[warp][lane] = cnt;
    }
    __syncthreads();
    {   // warp w turns the chunk counts of column w into an exclusive prefix over the row chunks (lane = row chunk)
        const int cnt = col_chunk[lane][warp];
        int incl = cnt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += n;
        }
        col_chunk[lane][warp] = incl - cnt;
        if (lane == 31) s_col_total[warp] = incl;
    }
    __syncthreads();
    // three independent jobs on the column totals, one warp each
    if (warp == 0) {
        const int total = s_col_total[lane];
        int incl = total;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += n;
        }
        s_col_ptr[lane] = incl - total;
        if (lane == 31) s_col_ptr[32] = incl;
        if (lane < C) col_ptr[lane] = incl - total;
        if (lane == C - 1) col_ptr[C] = incl;
    } else if (warp == 1) {
        // column order, heaviest first (stable)
        const int total = s_col_total[lane];
        int rank = 0;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int other = __shfl_sync(0xffffffffu, total, j);
            rank += (j < C) && ((other > total) || (other == total && j < lane));
        }
        if (lane < C) col_order[rank] = lane;
    } else if (warp == 2) {
        int mxc = lane < C ? s_col_total[lane] : 0;
#pragma unroll
        for (int d = 16; d; d >>= 1) mxc = max(mxc, __shfl_xor_sync(0xffffffffu, mxc, d));
        if (lane == 0) {
            header[H_NNZ] = nnz;
            header[H_SDD_ITEMS] = n_items;
            header[H_NDROP] = R * C - nnz;
            header[H_R] = R;
            header[H_C] = C;
            header[H_MAX_ROW] = s_max_row;
            header[H_MAX_COL] = mxc;
            if (a.counter) {                                      // every thread read it before the first barrier
                const unsigned long long drawn = offset - a.offset;
                if (!a.batch_arrivals) {
                    *a.counter = drawn + 1;
                } else {
                    // every CTA of the batch read the counter before it arrives here; the last one moves it on
                    __threadfence();
                    if (atomicAdd(a.batch_arrivals, 1u) == unsigned(a.batch_n - 1)) {
                        *a.counter = drawn + a.batch_n;
                        *a.batch_arrivals = 0u;
                    }
                }
            }
        }
    }
    __syncthreads();
    if (lane < C) {
        int off = s_col_ptr[lane] + col_chunk[warp][lane];
        for (int r = cr0; r < cr1; ++r)
            if ((keepmask[r] >> lane) & 1u) row_idx[off++] = r;
    }

    // ---- row order, heaviest first (stable rank sort for short lists, counting sort otherwise)
    if (R <= 64) {
        if (int(threadIdx.x) < R) {
            const int mine = __popc(keepmask[threadIdx.x]);
            int rank = 0;
            for (int j = 0; j < R; ++j) {
                const int other = __popc(keepmask[j]);
                rank += (other > mine) || (other == mine && j < int(threadIdx.x));
            }
            row_order[rank] = threadIdx.x;
        }
    } else {
        // counting sort on the kept count (at most 33 bins); lanes of a warp that share a bin add to it once
        const int rounds = (R + kPlanThreads - 1) / kPlanThreads;
        for (int k = 0; k < rounds; ++k) {
            const int r = k * kPlanThreads + threadIdx.x;
            const unsigned live = __ballot_sync(0xffffffffu, r < R);
            if (r < R) {
                const int key = C - __popc(keepmask[r]);
                const unsigned peers = __match_any_sync(live, key);
                if (lane == __ffs(peers) - 1) atomicAdd(&bins[key], __popc(peers));
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int run = 0;
            for (int k = 0; k <= C; ++k) { const int c = bins[k]; bins[k] = run; run += c; }
        }
        __syncthreads();
        for (int k = 0; k < rounds; ++k) {
            const int r = k * kPlanThreads + threadIdx.x;
            const unsigned live = __ballot_sync(0xffffffffu, r < R);
            if (r < R) {
                const int key = C - __popc(keepmask[r]);
                const unsigned peers = __match_any_sync(live, key);
                const int leader = __ffs(peers) - 1;
                int base = 0;
                if (lane == leader) base = atomicAdd(&bins[key], __popc(peers));
                base = __shfl_sync(peers, base, leader);
                row_order[base + __popc(peers & ((1u << lane) - 1u))] = r;
            }
        }
    }
}

__global__ void __launch_bounds__(kPlanThreads, 1) plan_bits_kernel(PlanArgs a) { plan_bits_body(a); }

// Several plans from one launch: CTA j builds the plan list[j] describes.  A training step draws one mask per
// SparseDrop layer; as separate launches of a few microseconds each they add up to a visible share of a small model's
// step, and nothing orders them among themselves, so they run side by side here.
__global__ void __launch_bounds__(kPlanThreads, 1) plan_bits_batch_kernel(const PlanArgs* __restrict__ list) {
    const PlanArgs a = list[blockIdx.x];
    plan_bits_body(a);
}

// The same plan from a cluster of kPlanClusterSize CTAs, for grids of thousands of tiles, where one SM is bound by
// the instructions it has to issue (a Philox draw and three list entries per tile).  CTA g owns a contiguous slice
// of the rows and does everything plan_bits_kernel does on that slice; what one slice must know of the others -
// kept tiles, work items, kept tiles per column and rows per kept count in the slices before it, and the totals -
// is exchanged once through distributed shared memory.
constexpr int kPlanClusterSize = 8;

struct PlanSliceTotals {
    int nnz, items, max_row;
    int col[32];      // kept tiles of the slice in each column
    int bins[34];     // rows of the slice by C - kept count
};

__global__ void __launch_bounds__(kPlanThreads, 1) plan_bits_cluster_kernel(PlanArgs a) {
    __shared__ unsigned keepmask[kBitsMaxRows];
    __shared__ int s_row_ptr[kBitsMaxRows];
    __shared__ int s_item_ptr[kBitsMaxRows];
    __shared__ unsigned long long pair_sums[33];
    __shared__ int col_chunk[32][33];
    __shared__ int s_col_base[32];
    __shared__ int bins[40];
    __shared__ PlanSliceTotals mine;
    __shared__ int s_base[4];          // kept tiles / work items before this slice; kept tiles / items of all slices

    cg::cluster_group cluster = cg::this_cluster();
    const int G = int(cluster.num_blocks()), gi = int(cluster.block_rank());
    const int R = a.R, C = a.C, rep = a.rep, rep_c = a.rep_c;
    const int Cm = (C + rep_c - 1) / rep_c;
    const int r_lo = int((long long)R * gi / G), r_hi = int((long long)R * (gi + 1) / G), Rn = r_hi - r_lo;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const sd_plan_layout L = plan_layout(R, C);
    int* header = reinterpret_cast<int*>(a.plan + L.header);
    int* row_ptr = reinterpret_cast<int*>(a.plan + L.row_ptr);
    int* col_idx = reinterpret_cast<int*>(a.plan + L.col_idx);
    int* col_ptr = reinterpret_cast<int*>(a.plan + L.col_ptr);
    int* row_idx = reinterpret_cast<int*>(a.plan + L.row_idx);
    int* kept_pairs = reinterpret_cast<int*>(a.plan + L.kept_pairs);
    int* drop_pairs = reinterpret_cast<int*>(a.plan + L.drop_pairs);
    int* row_order = reinterpret_cast<int*>(a.plan + L.row_order);
    int* col_order = reinterpret_cast<int*>(a.plan + L.col_order);
    int* sdd_items = reinterpret_cast<int*>(a.plan + L.sdd_items);
    unsigned char* gmask = a.plan + L.mask;
    grid_dep_launch();
    grid_dep_wait();   // the counter, a caller's mask and the plan buffer may belong to the previous kernel
    const unsigned long long offset = a.offset + (a.counter ? *a.counter : 0ull);
    if (threadIdx.x == 0) mine.max_row = 0;
    if (threadIdx.x < 34) mine.bins[threadIdx.x] = 0;

    // ---- the drop decisions of the slice, one tile per thread; kept tiles set their bit in the row word
    for (int r = threadIdx.x; r < Rn; r += kPlanThreads) keepmask[r] = 0u;
    __syncthreads();
    for (int i = threadIdx.x; i < Rn * C; i += kPlanThreads) {
        const int rl = i / C, c = i - rl * C, r = r_lo + rl;
        const int lr = r / rep, lc = c / rep_c;
        bool drop;
        if (a.from_seed) {
            drop = philox_drop(a.seed, offset, (unsigned long long)lr * Cm + lc, a.p);
            if (a.mask_out && r == lr * rep && c == lc * rep_c) a.mask_out[(long long)lr * Cm + lc] = drop;
        } else {
            drop = a.mask_in[lr * a.mask_rs + lc * a.mask_cs] != 0;
        }
        gmask[(long long)r * C + c] = drop;
        if (!drop) atomicOr(&keepmask[rl], 1u << c);
    }
    __syncthreads();

    // ---- offsets of the slice's rows relative to the slice: thread t owns rows [t*rpt, (t+1)*rpt) of it
    {
        const int rpt = (Rn + kPlanThreads - 1) / kPlanThreads;
        const int r0 = min(Rn, int(threadIdx.x) * rpt), r1 = min(Rn, r0 + rpt);
        int kept = 0, items = 0, mx = 0;
        for (int r = r0; r < r1; ++r) {
            const int cnt = __popc(keepmask[r]);
            kept += cnt;
            items += (cnt + 1) >> 1;
            mx = max(mx, cnt);
        }
        int kept_off, item_off, nnz, n_items;
        block_exclusive_scan_pair(kept, items, pair_sums, kept_off, item_off, nnz, n_items);
        if (mx) atomicMax(&mine.max_row, mx);
        for (int r = r0; r < r1; ++r) {
            const int cnt = __popc(keepmask[r]);
            s_row_ptr[r] = kept_off;
            s_item_ptr[r] = item_off;
            kept_off += cnt;
            item_off += (cnt + 1) >> 1;
        }
        if (threadIdx.x == 0) { mine.nnz = nnz; mine.items = n_items; }
    }
    // ---- kept tiles per column: warp w counts the row chunk [w*rpw, (w+1)*rpw) of the slice; lane = column
    const int rpw = (Rn + 31) / 32;
    const int cr0 = min(Rn, warp * rpw), cr1 = min(Rn, cr0 + rpw);
    {
        int cnt = 0;
        for (int r = cr0; r < cr1; ++r) cnt += (keepmask[r] >> lane) & 1u;
        col_chunk[warp][lane] = cnt;
    }
    // ---- rows of the slice by kept count (lanes of a warp that share a count add to it once)
    const int rounds = (Rn + kPlanThreads - 1) / kPlanThreads;
    for (int k = 0; k < rounds; ++k) {
        const int r = k * kPlanThreads + threadIdx.x;
        const unsigned live = __ballot_sync(0xffffffffu, r < Rn);
        if (r < Rn) {
            const int key = C - __popc(keepmask[r]);
            const unsigned peers = __match_any_sync(live, key);
            if (lane == __ffs(peers) - 1) atomicAdd(&mine.bins[key], __popc(peers));
        }
    }
    __syncthreads();
    {   // warp w turns the chunk counts of column w into an exclusive prefix over the row chunks (lane = row chunk)
        const int cnt = col_chunk[lane][warp];
        int incl = cnt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += n;
        }
        col_chunk[lane][warp] = incl - cnt;
        if (lane == 31) mine.col[warp] = incl;
    }
    cluster.sync();    // every slice's totals are complete and visible to the whole cluster

    // ---- what the other slices contribute
    if (warp == 0) {
        int before = 0, all = 0;                     // column `lane`
        for (int g = 0; g < G; ++g) {
            const int v = cluster.map_shared_rank(&mine, g)->col[lane];
            if (g < gi) before += v;
            all += v;
        }
        int incl = all;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += n;
        }
        s_col_base[lane] = incl - all + before;      // where this slice's rows start in column `lane`'s list
        if (gi == 0) {
            if (lane < C) col_ptr[lane] = incl - all;
            if (lane == C - 1) col_ptr[C] = incl;
            int rank = 0;                            // column order, heaviest first (stable)
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int other = __shfl_sync(0xffffffffu, all, j);
                rank += (j < C) && ((other > all) || (other == all && j < lane));
            }
            if (lane < C) col_order[rank] = lane;
            int mxc = lane < C ? all : 0;
#pragma unroll
            for (int d = 16; d; d >>= 1) mxc = max(mxc, __shfl_xor_sync(0xffffffffu, mxc, d));
            if (lane == 0) header[H_MAX_COL] = mxc;
        }
    } else if (warp == 1) {
        // rows by kept count: bin `lane` (and bin 32 by lane 0 on a second turn) of all slices
        int start_here = 0;
        for (int turn = 0; turn < 2; ++turn) {
            const int key = turn * 32 + lane;
            int before = 0, all = 0;
            if (key <= C)
                for (int g = 0; g < G; ++g) {
                    const int v = cluster.map_shared_rank(&mine, g)->bins[key];
                    if (g < gi) before += v;
                    all += v;
                }
            int incl = all;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += n;
            }
            if (key <= C) bins[key] = start_here + incl - all + before;
            start_here += __shfl_sync(0xffffffffu, incl, 31);
        }
    } else if (warp == 2 && lane == 0) {
        int nnz_before = 0, items_before = 0, nnz_all = 0, items_all = 0, max_row = 0;
        for (int g = 0; g < G; ++g) {
            const PlanSliceTotals* t = cluster.map_shared_rank(&mine, g);
            if (g < gi) { nnz_before += t->nnz; items_before += t->items; }
            nnz_all += t->nnz;
            items_all += t->items;
            max_row = max(max_row, t->max_row);
        }
        s_base[0] = nnz_before; s_base[1] = items_before; s_base[2] = nnz_all; s_base[3] = items_all;
        if (gi == 0) {
            header[H_NNZ] = nnz_all;
            header[H_SDD_ITEMS] = items_all;
            header[H_NDROP] = R * C - nnz_all;
            header[H_R] = R;
            header[H_C] = C;
            header[H_MAX_ROW] = max_row;
            row_ptr[R] = nnz_all;
            if (a.counter) *a.counter = offset - a.offset + 1;   // every CTA read it before the cluster barrier
        }
    }
    cluster.sync();    // nobody reads another CTA's shared memory after this point; also a CTA-wide barrier

    // ---- row lists of the slice, one tile per thread: positions are popcounts of the row word below this column
    const int nnz_before = s_base[0], items_before = s_base[1];
    for (int r = threadIdx.x; r < Rn; r += kPlanThreads) row_ptr[r_lo + r] = nnz_before + s_row_ptr[r];
    for (int i = threadIdx.x; i < Rn * C; i += kPlanThreads) {
        const int rl = i / C, c = i - rl * C, r = r_lo + rl;
        const unsigned mask = keepmask[rl];
        const int base = nnz_before + s_row_ptr[rl];
        const int j = __popc(mask & ((1u << c) - 1u));           // kept tiles left of this column
        if ((mask >> c) & 1u) {
            col_idx[base + j] = c;
            *reinterpret_cast<int2*>(kept_pairs + 2 * (base + j)) = make_int2(r, c);
            if ((j & 1) == 0) {                                  // first tile of a pair: its partner is the next kept column
                const unsigned above = c == 31 ? 0u : mask & ~((2u << c) - 1u);
                int* it = sdd_items + 3 * (items_before + s_item_ptr[rl] + (j >> 1));
                it[0] = r;
                it[1] = c;
                it[2] = above ? __ffs(above) - 1 : -1;
            }
        } else {
            const int d = r * C - base + (c - j);                // dropped tiles before this one
            *reinterpret_cast<int2*>(drop_pairs + 2 * d) = make_int2(r, c);
        }
    }
    // ---- column lists: warp = row chunk of the slice, lane = column
    if (lane < C) {
        int off = s_col_base[lane] + col_chunk[warp][lane];
        for (int r = cr0; r < cr1; ++r)
            if ((keepmask[r] >> lane) & 1u) row_idx[off++] = r_lo + r;
    }
    // ---- row order, heaviest first: counting sort on the kept count, the bins already offset for this slice
    for (int k = 0; k < rounds; ++k) {
        const int r = k * kPlanThreads + threadIdx.x;
        const unsigned live = __ballot_sync(0xffffffffu, r < Rn);
        if (r < Rn) {
            const int key = C - __popc(keepmask[r]);
            const unsigned peers = __match_any_sync(live, key);
            const int leader = __ffs(peers) - 1;
            int base = 0;
            if (lane == leader) base = atomicAdd(&bins[key], __popc(peers));
            base = __shfl_sync(peers, base, leader);
            row_order[base + __popc(peers & ((1u << lane) - 1u))] = r_lo + r;
        }
    }
}

static int launch_plan(const PlanArgs& a, void* stream) {
    if (!a.plan) return fail(SD_ERR_INVALID_ARG, "plan buffer is null");
    if (a.R <= 0 || a.C <= 0) return fail(SD_ERR_INVALID_ARG, "plan grid must be positive (R=%d, C=%d)", a.R, a.C);
    if (a.rep <= 0 || a.rep_c <= 0) return fail(SD_ERR_INVALID_ARG, "block_size must be a positive multiple of 128");
    if (int64_t(a.R) * a.C > (int64_t(1) << 26))
        return fail(SD_ERR_TOO_LARGE, "plan grid %d x %d exceeds 2^26 tiles", a.R, a.C);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(kPlanThreads);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    static const int cluster_min_tiles = [] {
        const char* e = getenv("SD_PLAN_CLUSTER_MIN_TILES");   // tuning knob: smallest grid that gets the cluster kernel
        return e ? atoi(e) : 1024;      // below ~1000 tiles the single CTA (4-6 us) beats the cluster's ~6.3 us floor
    }();
    static const int cluster_min_rows = [] {
        const char* e = getenv("SD_PLAN_CLUSTER_MIN_ROWS");
        return e ? atoi(e) : 8 * kPlanClusterSize;
    }();
    if (a.C <= 32 && a.R >= cluster_min_rows && a.R >= kPlanClusterSize && int64_t(a.R) * a.C >= cluster_min_tiles &&
        a.R <= kBitsMaxRows * kPlanClusterSize) {
        // thousands of tiles: a cluster of CTAs, each with a slice of the rows
        cudaLaunchAttribute cattr[2];
        cattr[0] = attr[0];
        cattr[1].id = cudaLaunchAttributeClusterDimension;
        cattr[1].val.clusterDim.x = kPlanClusterSize;
        cattr[1].val.clusterDim.y = 1;
        cattr[1].val.clusterDim.z = 1;
        cfg.gridDim = dim3(kPlanClusterSize);
        cfg.attrs = cattr;
        cfg.numAttrs = 2;
        SD_CUDA_TRY(cudaLaunchKernelEx(&cfg, plan_bits_cluster_kernel, a));
    } else if (a.C <= 32 && a.R <= kBitsMaxRows)
        SD_CUDA_TRY(cudaLaunchKernelEx(&cfg, plan_bits_kernel, a));
    else
        SD_CUDA_TRY(cudaLaunchKernelEx(&cfg, plan_kernel, a));
    return SD_OK;
}

}  // namespace sd

extern "C" {


size_t sd_plan_bytes(int R, int C) {
    if (R <= 0 || C <= 0) return 0;
    return size_t(sd::plan_layout(R, C).total_bytes);
}

int sd_plan_offsets(int R, int C, sd_plan_layout* out) {
    if (!out || R <= 0 || C <= 0) return sd::fail(SD_ERR_INVALID_ARG, "sd_plan_offsets: bad arguments");
    *out = sd::plan_layout(R, C);
    return SD_OK;
}

int sd_plan_from_seed(void* plan, int R, int C, int rep_r, int rep_c, uint64_t seed, uint64_t offset, float p,
                      uint8_t* mask_out, void* stream) {
    if (!(p >= 0.0f && p < 1.0f)) return sd::fail(SD_ERR_INVALID_ARG, "Dropout probability must be in [0, 1)");
    sd::PlanArgs a{};
    a.plan = static_cast<unsigned char*>(plan);
    a.R = R; a.C = C; a.rep = rep_r; a.rep_c = rep_c;
    a.from_seed = 1;
    a.seed = seed; a.offset = offset; a.p = p;
    a.mask_out = mask_out;
    return sd::launch_plan(a, stream);
}

int sd_plan_from_seed_counter(void* plan, int R, int C, int rep_r, int rep_c, uint64_t seed, uint64_t base_offset,
                              uint64_t* device_counter, float p, uint8_t* mask_out, void* stream) {
    if (!(p >= 0.0f && p < 1.0f)) return sd::fail(SD_ERR_INVALID_ARG, "Dropout probability must be in [0, 1)");
    if (!device_counter) return sd::fail(SD_ERR_INVALID_ARG, "device_counter is null");
    sd::PlanArgs a{};
    a.plan = static_cast<unsigned char*>(plan);
    a.R = R; a.C = C; a.rep = rep_r; a.rep_c = rep_c;
    a.from_seed = 1;
    a.seed = seed; a.offset = base_offset; a.p = p;
    a.counter = reinterpret_cast<unsigned long long*>(device_counter);
    a.mask_out = mask_out;
    return sd::launch_plan(a, stream);
}

size_t sd_plan_batch_desc_bytes(int n) {
    return n > 0 ? size_t(n) * sizeof(sd::PlanArgs) + 16 : 0;     // descriptors, then the arrival counter
}

int sd_plan_batch_describe(void* host_desc, void* device_desc, int n, int i, void* plan, int R, int C, int rep_r, int rep_c,
                           uint64_t seed, uint64_t base_offset, uint64_t* device_counter, float p, uint8_t* mask_out) {
    if (!host_desc || !device_desc || n <= 0 || i < 0 || i >= n) return sd::fail(SD_ERR_INVALID_ARG, "bad batch descriptor arguments");
    if (!(p >= 0.0f && p < 1.0f)) return sd::fail(SD_ERR_INVALID_ARG, "Dropout probability must be in [0, 1)");
    if (!plan || !device_counter) return sd::fail(SD_ERR_INVALID_ARG, "plan or device_counter is null");
    if (R <= 0 || C <= 0 || rep_r <= 0 || rep_c <= 0) return sd::fail(SD_ERR_INVALID_ARG, "plan grid and block repeat must be positive");
    if (C > 32 || R > sd::kBitsMaxRows)
        return sd::fail(SD_ERR_TOO_LARGE, "a batched plan is at most %d x 32 tiles (got %d x %d)", sd::kBitsMaxRows, R, C);
    sd::PlanArgs a{};
    a.plan = static_cast<unsigned char*>(plan);
    a.R = R; a.C = C; a.rep = rep_r; a.rep_c = rep_c;
    a.from_seed = 1;
    a.seed = seed; a.offset = base_offset + uint64_t(i); a.p = p;
    a.counter = reinterpret_cast<unsigned long long*>(device_counter);
    a.mask_out = mask_out;
    a.batch_arrivals = reinterpret_cast<unsigned int*>(static_cast<unsigned char*>(device_desc) + size_t(n) * sizeof(sd::PlanArgs));
    a.batch_n = n;
    static_cast<sd::PlanArgs*>(host_desc)[i] = a;
    return SD_OK;
}

int sd_plan_batch_launch(const void* device_desc, int n, void* stream) {
    if (!device_desc || n <= 0) return sd::fail(SD_ERR_INVALID_ARG, "bad batch launch arguments");
    if (reinterpret_cast<uintptr_t>(device_desc) & 7) return sd::fail(SD_ERR_LAYOUT, "descriptors must be 8-byte aligned");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n);
    cfg.blockDim = dim3(sd::kPlanThreads);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    SD_CUDA_TRY(cudaLaunchKernelEx(&cfg, sd::plan_bits_batch_kernel, static_cast<const sd::PlanArgs*>(device_desc)));
    return SD_OK;
}

int sd_plan_from_mask(void* plan, int R, int C, int rep_r, int rep_c, const uint8_t* mask, int64_t mask_row_stride,
                      int64_t mask_col_stride, void* stream) {
    if (!mask) return sd::fail(SD_ERR_INVALID_ARG, "mask is null");
    sd::PlanArgs a{};
    a.plan = static_cast<unsigned char*>(plan);
    a.R = R; a.C = C; a.rep = rep_r; a.rep_c = rep_c;
    a.from_seed = 0;
    a.mask_in = mask;
    a.mask_rs = mask_row_stride; a.mask_cs = mask_col_stride;
    return sd::launch_plan(a, stream);
}

}  // extern "C"
