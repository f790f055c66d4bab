// Persistent, warp-specialised tcgen05 GEMM for sm_100a that walks only kept tiles.
//
// One kernel template serves the three products of a SparseDrop linear layer and the dense
// comparator; D[MM, NN] = scale * A[MM, KK] . B[NN, KK]^T throughout:
//   dense : every 128-wide K tile                      (flash_dropout/cuda/src/gemm.cuh:100-140)
//   DSD   : per 128-row block of A, only the K tiles on that block's kept list
//           (flash_dropout/cuda/src/matmul_dsd.cuh:18-68 re-reads a bool mask every k-step and
//           `continue`s; here the producer warp never even visits a dropped tile)
//   SDD   : only kept 128x128 output tiles are computed, two per work item (one per item when
//           that would leave half the SMs idle); dropped tiles are zero-filled by the otherwise
//           idle epilogue warps
//           (flash_dropout/cuda/src/matmul_sdd.cuh:18-67 launches a CTA per tile, kept or not)
//
// CTA = 7 or 11 warps on one SM, 128 x 256 output tile, 64-wide K stages in a 4-deep TMA ring:
//   warp 0 and the last warp
//             producers: one lane of each issues cp.async.bulk.tensor loads (no multicast) into
//                        128B-swizzled shared memory - warp 0 the A tiles, the last warp the B tiles
//                        (one thread issues a load only every ~110 cycles) - completion on `full`
//                        mbarriers
//   warp 1    MMA      : one lane issues tcgen05.mma (M128 N256 K16, fp32 accumulate in TMEM),
//                        tcgen05.commit releases ring stages and publishes accumulators
//   warps 2-9 epilogue : tcgen05.ld the accumulator (two 256-column TMEM buffers, so the
//                        epilogue of tile i overlaps the main loop of tile i+1), scale, convert,
//                        stage in shared memory, TMA-store to global memory.  Two warps per TMEM
//                        lane quadrant, each with half of the tile's columns: with a short reduction
//                        (K of a few hundred) the epilogue of a tile takes as long as its main loop
// Both operands may be K-major (reduction dimension contiguous) or MN-major; that is the
// (row|col)-major x (row|col)-major operand matrix of flash_dropout/cuda/src/gemm_binding.cu:51-53.
//
// Scheduling.  With several output tiles per SM, whole tiles are dealt round-robin from a list sorted
// heaviest row block first.  With fewer tiles than SMs and a long reduction (the dW product of a layer fed
// thousands of rows, or of a conv whose reduction runs over all N*P*Q pixels) every output tile gets a group
// of consecutive CTAs instead: one each, and the spare CTAs dealt out in proportion to the tiles' kept K
// tiles, so every SM gets about the same number of MMA steps.  Each CTA of a group computes one contiguous
// part of the tile's kept K-tile list, parks its fp32 accumulator in its workspace slot and counts itself in;
// it then waits, bounded, for the rest of the group and adds up ITS share of the tile's 32x32 units over all
// parked accumulators, in CTA order (so results do not depend on timing), and stores them.  The CTA that
// finishes last clears the counters.  This needs the caller's workspace; without one, whole tiles are used
// throughout.
//
// Every wait is bounded (sd_ptx.cuh: mbar_wait); on expiry the CTA records a code in the status
// word, every role leaves its loop, TMEM is freed and the kernel returns normally.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstdlib>
#include <mutex>

#include "sd_common.h"
#include "sd_plan.cuh"
#include "sd_ptx.cuh"

namespace sd {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_BYTES = BN * BK * 2;        // 32 KiB
constexpr int B_HALF_BYTES = B_BYTES / 2;   // one 128-row half of the B tile
constexpr int MN_ATOM_BYTES = 64 * BK * 2;  // 64 MN-elements x 64 K-rows, one MN-major TMA box
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TILE_SMEM = STAGES * STAGE_BYTES;          // 192 KiB
// Epilogue warps: four (one per TMEM lane quadrant, two staging buffers each) or eight (two per quadrant, each with
// half of a tile's columns and one staging buffer); the launch's block size says which.  Eight shorten the epilogue
// of a tile, which decides short reductions (K of a few hundred: the epilogue takes as long as the main loop) and
// small launches (one tile per CTA, nothing to hide the epilogue behind); with a long reduction the four extra
// warps only take issue slots from the producer and MMA warps.
constexpr int MAX_EPI_WARPS = 8;
constexpr int STAGING_BYTES = 8 * 4096;                  // TMA-store staging
// Tile table: a CTA that runs several whole-tile passes resolves all of them once, in its prologue, into shared
// memory (row block, column tile, keep bits of the row block's K tiles), so that no role pays the chain of
// dependent index loads (order -> list bounds -> list entries) again for every tile.
constexpr int TAB_MAX = 96, TAB_MIN = 8;
constexpr int TAB_BYTES = TAB_MAX * 16;
constexpr int GEMM_SMEM = TILE_SMEM + 1024 /*align*/ + 256 /*barriers*/ + STAGING_BYTES + TAB_BYTES;
static_assert(GEMM_SMEM <= 227 * 1024, "over the shared memory of one CTA");
constexpr int GEMM_MAX_THREADS = 96 + MAX_EPI_WARPS * 32;   // producer A, MMA, epilogue warps, producer B
constexpr int GATHER_THREADS = 96 + 4 * 32 + 8 * 32;         // with gather warps: four epilogue warps, eight gather warps
constexpr int TMEM_COLS = 512;

// Workspace of the split schedule: flags first, then one fp32 partial tile per CTA.
constexpr int WS_MAX_CTAS = 1024;
constexpr size_t WS_FLAG_BYTES = 2 * WS_MAX_CTAS * sizeof(int);   // arrive[] then done[], indexed by the tile owner's CTA
constexpr size_t WS_SLOT_FLOATS = size_t(BM) * BN;
constexpr size_t WS_SLOT_BYTES = WS_SLOT_FLOATS * sizeof(float);   // 128 KiB; one slot per CTA

enum GemmMode { MODE_DENSE = 0, MODE_DSD = 1, MODE_SDD = 2 };
enum StatusCode { ST_PRODUCER = 1, ST_MMA_FULL = 2, ST_MMA_ACC = 3, ST_EPILOGUE = 4, ST_FIXUP = 5 };

// Geometry of a convolution whose im2col matrix (rows = output pixels m = (n, p, q), columns k = c*R*3 + r*3 + s,
// the unfold order of flash_dropout/functional/im2col_conv2d.py:17-20) is the A operand, built on the fly by the
// gather warps instead of being read through a tensor map.  Only filters 3 wide with unit horizontal stride and
// dilation and one column of padding (so Q == W) on rows of 8, 16, 32 or 64 pixels take this path.
struct ConvGather {
    const unsigned short* x;     // NCHW input, contiguous, 16-byte aligned
    int C, H, W, R, P;
    int stride_h, dil_h, pad_h;
    int PQ, HW;
    int k_real;                  // C * R * 3: columns of the im2col matrix that exist
    int pixels;                  // N * P * Q: rows that exist
    int log2_w;                  // W is a power of two
    uint32_t mul_pq, shr_pq;     // fast_div constants for P * Q and R
    uint32_t mul_r, shr_r;
    int pass_dc[3], pass_dr[3];  // (channel, filter row) step between a gather thread's passes, per GATHER mode:
                                 // the pair index advances by 4 (mode 1) or 8 (mode 2) = pass_dc * R + pass_dr
};

// n / d for 0 <= n < 2^31 by one multiply-high and a shift; (mul, shr) come from fast_div_constants(d).
__host__ __device__ __forceinline__ int fast_div(int n, uint32_t mul, uint32_t shr) {
#if defined(__CUDA_ARCH__)
    return mul ? int(__umulhi(uint32_t(n), mul) >> shr) : n;
#else
    return mul ? int((uint64_t(uint32_t(n)) * mul >> 32) >> shr) : n;
#endif
}
// Round-up multiplier: with L = ceil(log2 d), mul = ceil(2^(31+L) / d) fits 32 bits and
// floor(n * mul / 2^(31+L)) == floor(n / d) for every n below 2^31.  d == 1 is flagged by mul == 0.
inline void fast_div_constants(uint32_t d, uint32_t* mul, uint32_t* shr) {
    if (d <= 1) { *mul = 0; *shr = 0; return; }
    uint32_t L = 0;
    while ((1ull << L) < d) ++L;
    const uint32_t pw = 31 + L;
    *mul = uint32_t(((1ull << pw) + d - 1) / d);
    *shr = pw - 32;
}

struct GemmArgs {
    int mode;
    int MM, NN, KK;
    void* C;
    long long c_rs, c_cs;
    float scale;
    int is_bf16;
    int n_row_blocks, n_col_tiles;   // dense / DSD tile grid (128 x 256 tiles)
    const int* list_ptr;             // DSD: kept K-tile list of row block rb = list_idx[list_ptr[rb] .. list_ptr[rb+1])
    const int* list_idx;
    const int* order;                // DSD: row blocks sorted by kept count, heaviest first
    const int* h_nnz;                // DSD: plan header entries: kept tiles, and the largest kept count of a row block
    const int* h_max;
    const int* items;                // SDD: (row block, col tile 0, col tile 1 or -1); with sdd_single: kept (row, col) pairs
    const int* n_items;
    int sdd_single;                  // SDD with one kept 128x128 tile per item: 1 = the plan's (row, col) is the result's
                                     // tile (row, col); 2 = the plan describes the transposed result: tile (col, row);
                                     // 3 = transposed plan, two kept tiles of one plan column per item: item j of column
                                     // c = entries 2j, 2j+1 of the column's kept-row list (list_ptr / list_idx), so two
                                     // tiles of one result row block share the A tile and one 128x256 MMA
    const int* zero_pairs;           // SDD: dropped (row block, col tile) pairs
    const int* n_zero;
    int* status;
    uint32_t idesc256, idesc128;
    int a_panel_kg, c_panel_kg;      // > 0: A / C is the conv's im2col matrix stored in panels of 128 pixels, each panel
                                     // [kg][128] (kg a multiple of 64); the tensor map then describes [panels*kg][128]
    int split;                       // 1: equal unit ranges with fix-up (needs the workspace); 0: whole tiles
    int tma_store;                   // result written by TMA from a swizzled staging buffer: 1 row-major, 2 column-major
    float* ws_slots;
    int* ws_flags;
    const unsigned char* direct_mask;   // DSD launches in which a CTA gets only a few tiles: the plan's tile mask
    int dm_stride_rb, dm_stride_k;      // (1 = dropped), byte (row block rb, K tile k) at rb * dm_stride_rb + k * dm_stride_k.
                                        // A CTA then reads its row block's <= 32 mask bytes in one round trip instead of
                                        // walking order -> list bounds -> list entries (three dependent loads)
    int use_table;                   // whole-tile schedule whose tiles can be described by the shared-memory table
    int tab_min;                     // fewest passes of a CTA from which the table is used
    int all_halves;                  // whole-tile schedule of a launch that would leave most SMs idle: every tile is
                                     // handed out as two 128-wide halves, so twice as many SMs stream the operands
    int act;                         // epilogue: 1 = ReLU on the result (eval/mlp/model.py:33-38 applies it as a separate op)
    const unsigned short* mask_src;  // epilogue: result elements whose mask_src element is <= 0 are written as zeros: the
    long long mask_rs;               // derivative of a ReLU that produced the layer's input (row-major, same shape as C)
    int out_f32, out_acc;            // result stored as fp32 (optionally added to what C holds) instead of 16-bit
    ConvGather conv;                 // used by the GATHER variants of the kernel only
};

// The part [i0, i1) of one output tile's kept K-tile list that this CTA computes.
struct Seg {
    int a_row, b_row0, b_row1;   // element coordinates along the operands' MN dimension; b_row1 < 0: absent
    const int* klist;            // kept K-tile indices of the whole tile, or null for 0..nk-1
    int nk, i0, i1;
    int owner, parts, part;      // split schedule: first CTA of the tile's group, CTAs in the group, this CTA's place
    uint32_t bits;               // use_bits: bit kb set = K tile kb is kept (replaces klist; at most 32 K tiles)
    bool use_bits;
};

// The K tiles of one segment, in order.  List entries are fetched one step ahead of their use, so the load of the
// next entry is in flight while the current K tile is being processed.
struct KIter {
    const int* klist;
    int i, i1, pre;
    uint32_t bits;
    bool use_bits;
    __device__ __forceinline__ void init(const Seg& w) {
        use_bits = w.use_bits;
        bits = w.bits;
        klist = w.klist;
        i = w.i0;
        i1 = w.i1;
        pre = (!use_bits && klist && i < i1) ? __ldg(klist + i) : 0;
    }
    __device__ __forceinline__ bool next(int& kb) {
        if (use_bits) {
            if (!bits) return false;
            kb = __ffs(bits) - 1;
            bits &= bits - 1;
            return true;
        }
        if (i >= i1) return false;
        if (klist) {
            kb = pre;
            if (i + 1 < i1) pre = __ldg(klist + i + 1);
        } else {
            kb = i;
        }
        ++i;
        return true;
    }
};

// Walks this CTA's share of the launch.  Every role of the CTA runs its own copy and sees the same
// segments in the same order.  Two schedules:
//   split == 0 : whole output tiles, dealt round-robin from a list sorted heaviest row block first
//                (longest-processing-time order); the choice when there are several tiles per SM;
//   split == 1 : every output tile gets a group of consecutive CTAs, sized in proportion to the tile's
//                work, and each CTA of the group one contiguous part of the tile's kept K-tile list (see
//                the file header); the choice when there are fewer tiles than SMs and a long reduction.
struct WorkIter {
    int t, n_tiles, stride, pass;   // whole tiles: this CTA's index, tile count, gridDim.x, next pass
    int nk_uniform;              // dense / SDD: K tiles per output tile
    int full_per_row, n_full;    // whole tiles: full-width column tiles per row block, and in total
    int whole_entries, n_entries;   // whole tiles: list entries that are whole tiles, and all entries (see init)
    int sp_rb, sp_nt, sp_owner, sp_parts, sp_part;   // split: this CTA's one segment; sp_parts == 0: none
    bool split, snake;
    const int4* tab;             // shared-memory tile table (see TAB_MAX), or null: resolve every tile from the plan
    int passes;                  // whole tiles: passes over the entry list this grid makes
    bool direct;                 // DSD, few passes: tiles resolved from the plan's mask bytes (see GemmArgs::direct_mask)

    __device__ __forceinline__ int count(const GemmArgs& g, int r) const {
        return __ldg(g.list_ptr + r + 1) - __ldg(g.list_ptr + r);
    }
    // Work (in half-width K-tile steps) of all tiles before `tile`, tiles counted in row-block-major order.
    // A 256-wide tile step costs 2, the 128-wide last column tile of a ragged N costs 1.
    __device__ __forceinline__ unsigned work_before(const GemmArgs& g, int tile, int row_weight) const {
        if (g.mode == MODE_SDD) return unsigned(tile) * unsigned(nk_uniform);
        const int rb = tile / g.n_col_tiles, nt = tile - rb * g.n_col_tiles;
        if (g.mode == MODE_DENSE) return unsigned(rb * row_weight + 2 * nt) * unsigned(nk_uniform);
        unsigned w = unsigned(row_weight) * unsigned(__ldg(g.list_ptr + rb));
        if (nt) w += unsigned(2 * nt) * unsigned(count(g, rb));
        return w;
    }
    // First CTA of tile `tile`: one CTA per tile, the spare ones dealt in proportion to the work before it.
    __device__ __forceinline__ int group_start(const GemmArgs& g, int tile, int row_weight, unsigned total, int spare,
                                               bool fits32) const {
        const unsigned w = work_before(g, tile, row_weight);
        const unsigned extra = fits32 ? (unsigned(spare) * w) / total
                                      : unsigned((unsigned long long)spare * w / total);
        return tile + int(extra);
    }
    __device__ void init(const GemmArgs& g, int cta, int n_ctas, const int4* table) {
        split = g.split != 0;
        tab = nullptr;
        nk_uniform = (g.KK + 127) >> 7;
        if (g.mode == MODE_SDD && g.sdd_single == 3) {
            n_tiles = 0;
            for (int c = 0; c < g.n_row_blocks; ++c) n_tiles += (count(g, c) + 1) >> 1;
        } else {
            n_tiles = g.mode == MODE_SDD ? __ldg(g.n_items) : g.n_row_blocks * g.n_col_tiles;
        }
        t = cta;
        stride = n_ctas;
        pass = 0;
        // with equal tiles (dense, SDD, a mask that dropped nothing) plain round-robin keeps neighbouring CTAs on
        // neighbouring tiles in every pass; see below for unequal row blocks
        direct = false;
        snake = false;
        sp_rb = sp_nt = sp_owner = sp_part = 0;
        sp_parts = 0;
        const bool ragged = (g.n_col_tiles - 1) * BN + 128 >= g.NN;
        full_per_row = (ragged && g.n_col_tiles > 1) ? g.n_col_tiles - 1 : g.n_col_tiles;
        n_full = g.n_row_blocks * full_per_row;
        // Whole tiles fill the grid wave by wave.  When the last, partial wave holds at most half as many tiles as
        // there are CTAs, its tiles are handed out as two 128-wide halves each: twice as many SMs share that wave and
        // its length drops from one tile to one half tile (a half costs ~0.8 of a tile, its A operand is not halved,
        // so a fuller last wave is better left whole).  The halves need no exchange between CTAs.
        whole_entries = n_tiles;
        {
            const int waves = n_tiles / n_ctas, rest = n_tiles - waves * n_ctas;
            if (waves >= 1 && rest > 0 && 2 * rest <= n_ctas && !(g.mode == MODE_SDD && g.sdd_single))
                whole_entries = waves * n_ctas;
            if (g.all_halves) whole_entries = 0;
        }
        n_entries = whole_entries + 2 * (n_tiles - whole_entries);
        passes = (n_entries + n_ctas - 1) / n_ctas;
        direct = g.direct_mask != nullptr && !split && passes < g.tab_min;
        // alternate the direction only when row blocks differ in length (and there is more than one pass)
        if (g.mode == MODE_DSD && passes > 1) snake = __ldg(g.h_nnz) != g.n_row_blocks * __ldg(g.h_max);
        // the table costs a CTA-wide barrier and one chain of index loads up front: worth it from a handful of tiles per
        // CTA on (the short tiles of a conv), not for the three or four long tiles of a large square product
        if (g.use_table && !split && passes >= g.tab_min && passes <= TAB_MAX) tab = table;
        if (!split || n_tiles == 0 || n_tiles > n_ctas) return;
        const int row_weight = 2 * g.n_col_tiles - (ragged ? 1 : 0);
        const unsigned total = work_before(g, n_tiles, row_weight);
        if (total == 0) return;                                   // everything dropped: only zero-filling is left
        const int spare = n_ctas - n_tiles;
        const bool fits32 = (unsigned long long)total * unsigned(spare) <= 0xffffffffull;
        int lo = 0, hi = n_tiles - 1;                             // last tile whose group starts at or before this CTA
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (group_start(g, mid, row_weight, total, spare, fits32) <= cta) lo = mid; else hi = mid - 1;
        }
        const int first = group_start(g, lo, row_weight, total, spare, fits32);
        const int next_first = lo + 1 < n_tiles ? group_start(g, lo + 1, row_weight, total, spare, fits32) : n_ctas;
        if (g.mode == MODE_SDD) { sp_rb = lo; sp_nt = 0; }
        else { sp_rb = lo / g.n_col_tiles; sp_nt = lo - sp_rb * g.n_col_tiles; }
        const int nk = g.mode == MODE_DSD ? count(g, sp_rb) : nk_uniform;
        int parts = next_first - first;
        if (parts > nk) parts = nk;                               // never more CTAs on a tile than it has K tiles
        sp_owner = first;
        sp_part = cta - first;
        sp_parts = sp_part < parts ? parts : 0;
    }
    __device__ __forceinline__ void fill(const GemmArgs& g, Seg& s, int row_block, int n_tile) const {
        s.bits = 0;
        s.use_bits = false;
        if (g.mode == MODE_SDD && g.sdd_single == 3) {
            int idx = row_block, c = 0, beg = 0, n = 0;
            for (; c < g.n_row_blocks; ++c) {                    // which plan column the item falls into
                beg = __ldg(g.list_ptr + c);
                n = __ldg(g.list_ptr + c + 1) - beg;
                const int items_c = (n + 1) >> 1;
                if (idx < items_c) break;
                idx -= items_c;
            }
            s.a_row = c * 128;
            s.b_row0 = __ldg(g.list_idx + beg + 2 * idx) * 128;
            s.b_row1 = 2 * idx + 1 < n ? __ldg(g.list_idx + beg + 2 * idx + 1) * 128 : -1;
            s.nk = nk_uniform;
            s.klist = nullptr;
        } else if (g.mode == MODE_SDD && g.sdd_single) {
            const int pr = __ldg(g.items + 2 * row_block), pc = __ldg(g.items + 2 * row_block + 1);
            s.a_row = (g.sdd_single == 2 ? pc : pr) * 128;
            s.b_row0 = (g.sdd_single == 2 ? pr : pc) * 128;
            s.b_row1 = -1;
            s.nk = nk_uniform;
            s.klist = nullptr;
        } else if (g.mode == MODE_SDD) {
            const int mb = __ldg(g.items + 3 * row_block), c0 = __ldg(g.items + 3 * row_block + 1),
                      c1 = __ldg(g.items + 3 * row_block + 2);
            s.a_row = mb * 128;
            s.b_row0 = c0 * 128;
            s.b_row1 = c1 >= 0 ? c1 * 128 : -1;
            s.nk = nk_uniform;
            s.klist = nullptr;
        } else {
            s.a_row = row_block * 128;
            s.b_row0 = n_tile * BN;
            s.b_row1 = (n_tile * BN + 128 < g.NN) ? n_tile * BN + 128 : -1;
            if (g.mode == MODE_DSD) {
                const int beg = __ldg(g.list_ptr + row_block);
                s.nk = __ldg(g.list_ptr + row_block + 1) - beg;
                s.klist = g.list_idx + beg;
            } else {
                s.nk = nk_uniform;
                s.klist = nullptr;
            }
        }
    }
    // Whole-tile schedule: the segment of pass `ps` for this CTA, resolved from the plan; false if the pass holds nothing
    // for this CTA.  Pass j hands out entries [j*stride, (j+1)*stride) of the heaviest-first list; with unequal row
    // blocks, forwards on even passes and backwards on odd ones, so the CTA that got the heaviest tile of one pass gets
    // the lightest of the next.
    __device__ bool resolve(const GemmArgs& g, int ps, Seg& s) const {
        const int entry = ps * stride + (((ps & 1) && snake) ? stride - 1 - t : t);   // pass 0 does not wait for `snake`
        if (entry >= n_entries) return false;
        const int tile = entry < whole_entries ? entry : whole_entries + ((entry - whole_entries) >> 1);
        const int half = entry < whole_entries ? -1 : ((entry - whole_entries) & 1);
        if (g.mode == MODE_SDD) {
            fill(g, s, tile, 0);
        } else {
            // list order: row blocks heaviest first, and when the last column tile is only 128 wide (half the
            // work), all full-width tiles before all narrow ones, so that no CTA collects only full-width tiles
            int rbi, nt;
            if (tile < n_full) { rbi = tile / full_per_row; nt = tile - rbi * full_per_row; }
            else { rbi = tile - n_full; nt = g.n_col_tiles - 1; }
            if (direct) {
                // the kept K tiles come straight from the mask bytes of the row block (with one pass the order of the
                // tiles does not matter either)
                const int rb = (passes > 1 && g.order) ? __ldg(g.order + rbi) : rbi;
                const unsigned char* m = g.direct_mask + (long long)rb * g.dm_stride_rb;
                uint32_t bits = 0;
                for (int j = 0; j < nk_uniform; ++j) bits |= uint32_t(__ldg(m + (long long)j * g.dm_stride_k) == 0) << j;
                s.a_row = rb * 128;
                s.b_row0 = nt * BN;
                s.b_row1 = (nt * BN + 128 < g.NN) ? nt * BN + 128 : -1;
                s.klist = nullptr;
                s.use_bits = true;
                s.bits = bits;
                s.nk = __popc(bits);
            } else {
                fill(g, s, g.order ? __ldg(g.order + rbi) : rbi, nt);
            }
        }
        if (s.nk == 0) return false;          // empty row blocks are zero-filled by the epilogue warps
        if (half >= 0) {                      // one 128-wide half of a tile of the last wave
            if (s.b_row1 < 0) {
                if (half == 1) return false;  // the tile is only 128 wide: there is no second half
            } else {
                if (half == 1) s.b_row0 = s.b_row1;
                s.b_row1 = -1;
            }
        }
        s.i0 = 0;
        s.i1 = s.nk;
        s.owner = 0; s.parts = 1; s.part = 0;
        return true;
    }
    // Prologue of a CTA that uses the tile table: every thread resolves some of the passes.
    __device__ void fill_table(const GemmArgs& g, int4* table, int tid, int n_threads) const {
        for (int ps = tid; ps < passes; ps += n_threads) {
            Seg s;
            int4 e = make_int4(-1, 0, 0, 0);
            if (resolve(g, ps, s)) {
                uint32_t bits = 0;
                if (g.mode == MODE_DSD)
                    for (int j = 0; j < s.nk; ++j) bits |= 1u << __ldg(s.klist + j);
                e = make_int4(s.a_row, s.b_row0, s.b_row1, int(bits));
            }
            table[ps] = e;
        }
    }
    __device__ bool next(const GemmArgs& g, Seg& s) {
        if (!split) {
            if (tab) {
                for (; pass < passes; ++pass) {
                    const int4 e = tab[pass];
                    if (e.x < 0) continue;
                    s.a_row = e.x; s.b_row0 = e.y; s.b_row1 = e.z;
                    s.klist = nullptr;
                    s.use_bits = g.mode == MODE_DSD;
                    s.bits = uint32_t(e.w);
                    s.nk = s.use_bits ? __popc(s.bits) : nk_uniform;
                    s.i0 = 0;
                    s.i1 = s.nk;
                    s.owner = 0; s.parts = 1; s.part = 0;
                    ++pass;
                    return true;
                }
                return false;
            }
            for (; pass < passes; ++pass) {
                if (!resolve(g, pass, s)) continue;
                ++pass;
                return true;
            }
            return false;
        }
        if (sp_parts == 0) return false;
        fill(g, s, sp_rb, sp_nt);
        s.i0 = s.nk * sp_part / sp_parts;
        s.i1 = s.nk * (sp_part + 1) / sp_parts;
        s.owner = sp_owner; s.parts = sp_parts; s.part = sp_part;
        sp_parts = 0;                             // one segment per CTA
        return true;
    }
};

// ------------------------------------------------------------------ epilogue stores
__device__ __forceinline__ uint32_t pack2(float a, float b, int is_bf16) {
    if (is_bf16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ unsigned short cvt1(float a, int is_bf16) {
    if (is_bf16) return __bfloat16_as_ushort(__float2bfloat16_rn(a));
    return __half_as_ushort(__float2half_rn(a));
}

// Scales 32 fp32 values and packs them into 16 words of two 16-bit results (lower half = the earlier value).
// One branch around all sixteen conversions: fp32 -> 16-bit conversions issue at a fraction of the ALU rate, and a
// per-value choice between the two formats would run both.
__device__ __forceinline__ void convert_chunk(const uint32_t (&r)[32], float scale, int is_bf16, uint32_t (&p)[16]) {
    if (is_bf16) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;"
                         : "=r"(p[j])
                         : "f"(__uint_as_float(r[2 * j + 1]) * scale), "f"(__uint_as_float(r[2 * j]) * scale));
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            asm volatile("cvt.rn.f16x2.f32 %0, %1, %2;"
                         : "=r"(p[j])
                         : "f"(__uint_as_float(r[2 * j + 1]) * scale), "f"(__uint_as_float(r[2 * j]) * scale));
    }
}

// Thread holds 32 consecutive fp32 values of output row `row`, columns [col, col+32).
__device__ __forceinline__ void store_chunk(const GemmArgs& g, bool vec_ok, int row, int col, const uint32_t (&r)[32]) {
    if (row >= g.MM || col >= g.NN) return;
    unsigned short* C = static_cast<unsigned short*>(g.C);
    if (vec_ok && col + 32 <= g.NN) {
        uint4* dst = reinterpret_cast<uint4*>(C + (long long)row * g.c_rs + col);
        uint32_t p[16];
        convert_chunk(r, g.scale, g.is_bf16, p);
#pragma unroll
        for (int v = 0; v < 4; ++v) dst[v] = make_uint4(p[4 * v], p[4 * v + 1], p[4 * v + 2], p[4 * v + 3]);
    } else {
        // ragged edge, unaligned rows, or a column-major result (consecutive lanes = consecutive
        // rows, so a column-major store is a 64-byte contiguous segment per warp instruction)
        uint32_t p[16];
        convert_chunk(r, g.scale, g.is_bf16, p);
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col + j < g.NN)
                C[(long long)row * g.c_rs + (long long)(col + j) * g.c_cs] = (unsigned short)(p[j >> 1] >> (16 * (j & 1)));
    }
}

// The same for an fp32 result (a gradient written, or added, straight into an fp32 buffer).
__device__ __forceinline__ void store_chunk_f32(const GemmArgs& g, int row, int col, const uint32_t (&r)[32]) {
    if (row >= g.MM || col >= g.NN) return;
    float* C = static_cast<float*>(g.C);
    if (g.c_cs == 1 && (g.c_rs & 3) == 0 && (reinterpret_cast<uintptr_t>(g.C) & 15) == 0 && col + 32 <= g.NN) {
        float4* dst = reinterpret_cast<float4*>(C + (long long)row * g.c_rs + col);
#pragma unroll
        for (int v = 0; v < 8; ++v) {
            float4 o = make_float4(__uint_as_float(r[4 * v]) * g.scale, __uint_as_float(r[4 * v + 1]) * g.scale,
                                   __uint_as_float(r[4 * v + 2]) * g.scale, __uint_as_float(r[4 * v + 3]) * g.scale);
            if (g.out_acc) { const float4 old = dst[v]; o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
            dst[v] = o;
        }
    } else {
        // column-major result: consecutive lanes = consecutive rows, one 128-byte segment per warp store
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col + j < g.NN) {
                float* dst = C + (long long)row * g.c_rs + (long long)(col + j) * g.c_cs;
                const float v = __uint_as_float(r[j]) * g.scale;
                *dst = g.out_acc ? *dst + v : v;
            }
    }
}

// Zero a 128 x 128 output tile with 128 threads (tid in [0,128)): one half of the epilogue group.
__device__ __forceinline__ void zero_tile(const GemmArgs& g, bool vec_ok, bool vec_t_ok, int tid, int row0, int col0) {
    if (g.out_f32) {
        if (g.out_acc) return;                                   // adding nothing
        float* C32 = static_cast<float*>(g.C);
        if (g.c_rs == 1) {
            for (int j = 0; j < 128; ++j)
                if (row0 + tid < g.MM && col0 + j < g.NN) C32[(long long)(col0 + j) * g.c_cs + row0 + tid] = 0.f;
        } else {
            for (int i = 0; i < 128; ++i)
                if (row0 + i < g.MM && col0 + tid < g.NN) C32[(long long)(row0 + i) * g.c_rs + (long long)(col0 + tid) * g.c_cs] = 0.f;
        }
        return;
    }
    unsigned short* C = static_cast<unsigned short*>(g.C);
    if (vec_ok && row0 + 128 <= g.MM && col0 + 128 <= g.NN) {
        const int cchunk = tid & 15, rsub = tid >> 4;
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
            const int row = row0 + i * 8 + rsub;
            *reinterpret_cast<uint4*>(C + (long long)row * g.c_rs + col0 + cchunk * 8) = make_uint4(0, 0, 0, 0);
        }
    } else if (vec_t_ok && row0 + 128 <= g.MM && col0 + 128 <= g.NN) {
        const int rchunk = tid & 15, csub = tid >> 4;
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
            const int col = col0 + i * 8 + csub;
            *reinterpret_cast<uint4*>(C + (long long)col * g.c_cs + row0 + rchunk * 8) = make_uint4(0, 0, 0, 0);
        }
    } else if (g.c_rs == 1) {
        for (int j = 0; j < 128; ++j)
            if (row0 + tid < g.MM && col0 + j < g.NN) C[(long long)(col0 + j) * g.c_cs + row0 + tid] = 0;
    } else {
        for (int i = 0; i < 128; ++i)
            if (row0 + i < g.MM && col0 + tid < g.NN) C[(long long)(row0 + i) * g.c_rs + (long long)(col0 + tid) * g.c_cs] = 0;
    }
}

// ------------------------------------------------------------------ epilogue-group helpers
// Before a warp refills a TMA-store staging buffer: the store that last used it has read it.
__device__ __forceinline__ void wait_staging_free(bool two_bufs, int n_stores, int lane) {
    if (n_stores < (two_bufs ? 2 : 1)) return;
    if (lane == 0) {
        if (two_bufs) bulk_wait_read<1>(); else bulk_wait_read<0>();
    }
    __syncwarp();
}

// The epilogue warps synchronise on named barrier 1, never on barrier 0.
__device__ __forceinline__ void epilogue_sync(int n_threads) { asm volatile("bar.sync 1, %0;" ::"r"(n_threads) : "memory"); }
__device__ __forceinline__ bool epilogue_all(bool ok, int n_threads) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(r)
        : "r"(uint32_t(ok)), "r"(n_threads)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ void flag_set(int* flag, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(v) : "memory");
}
// Bounded wait for another CTA's flag (same limit and abort protocol as mbar_wait).
__device__ __forceinline__ bool flag_wait(const int* flag, volatile int* abort_flag, int* status, int code) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v != 0) return true;
        if ((it & 0xff) == 0xff) {
            if (*abort_flag) return false;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > kWaitLimitNs) {
                *abort_flag = 1;
                if (status) atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}


// ------------------------------------------------------------------ shared tiles of the split schedule
// The CTAs seg.owner .. seg.owner + seg.parts - 1 have each parked the partial accumulator of their part of one
// output tile in their workspace slot and counted themselves in arrive[owner].  Once the count is complete, every
// one of them adds up a different share of the tile's 32x32 units over all partials, in CTA order (so the result
// does not depend on timing), scales, converts and stores it.  The last one to finish clears the two counters,
// which leaves the workspace ready for the next launch.
__device__ bool reduce_shared_tile(const GemmArgs& g, const Seg& seg, int eidx, int epi_threads, volatile int* abort_flag) {
    const int owner = seg.owner, P = seg.parts, my_index = seg.part;
    const int last = owner + P - 1;
    int* arrive = g.ws_flags + owner;
    int* done = g.ws_flags + WS_MAX_CTAS + owner;
    bool ok = true;
    if (eidx == 0) ok = counter_wait(arrive, P, abort_flag, g.status, ST_FIXUP);
    if (!epilogue_all(ok, epi_threads)) return false;
    const int n_units = (seg.b_row1 >= 0 ? 8 : 4) * 4;
    unsigned short* C = static_cast<unsigned short*>(g.C);
    const bool quad_ok = g.c_cs == 1 && (g.c_rs & 3) == 0 && (reinterpret_cast<uintptr_t>(g.C) & 7) == 0;
    // A unit is 8 four-column pieces x 32 rows of 16 bytes, shared by all epilogue threads.  The loads of four partial
    // tiles are kept in flight at once, so the depth of the dependent chain is P / 4 round trips.
    for (int uu = my_index; uu < n_units; uu += P) {
      const int c = uu >> 2, q = uu & 3;
      for (int e = eidx; e < 256; e += epi_threads) {            // piece index inside the unit: [4-column piece][row]
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const size_t unit_off = size_t(uu) * 1024 + size_t(e) * 4;
        int pc = owner;
        while (pc <= last) {
            const float4* src[4];
            int n = 0;
            for (; pc <= last && n < 4; ++pc)
                src[n++] = reinterpret_cast<const float4*>(g.ws_slots + size_t(pc) * WS_SLOT_FLOATS + unit_off);
            float4 v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (i < n) v[i] = __ldcg(src[i]);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (i < n) { acc.x += v[i].x; acc.y += v[i].y; acc.z += v[i].z; acc.w += v[i].w; }
        }
        const int row = seg.a_row + q * 32 + (e & 31);
        const int col = (c < 4 ? seg.b_row0 + c * 32 : seg.b_row1 + (c - 4) * 32) + (e >> 5) * 4;
        if (row >= g.MM || col >= g.NN) continue;
        float f[4] = {acc.x * g.scale, acc.y * g.scale, acc.z * g.scale, acc.w * g.scale};
        if (g.act == 1) {
#pragma unroll
            for (int j = 0; j < 4; ++j) f[j] = fmaxf(f[j], 0.f);
        }
        if (g.out_f32) {
            float* C32 = static_cast<float*>(g.C);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (col + j < g.NN) {
                    float* dst = C32 + (long long)row * g.c_rs + (long long)(col + j) * g.c_cs;
                    *dst = g.out_acc ? *dst + f[j] : f[j];
                }
        } else if (quad_ok && col + 4 <= g.NN) {
            uint2 o;
            o.x = pack2(f[0], f[1], g.is_bf16);
            o.y = pack2(f[2], f[3], g.is_bf16);
            *reinterpret_cast<uint2*>(C + (long long)row * g.c_rs + col) = o;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (col + j < g.NN) C[(long long)row * g.c_rs + (long long)(col + j) * g.c_cs] = cvt1(f[j], g.is_bf16);
        }
      }
    }
    epilogue_sync(epi_threads);                                  // every thread has read its share
    if (eidx == 0) {
        __threadfence();
        if (atomicAdd(done, 1) == P - 1) {
            flag_set(arrive, 0);
            flag_set(done, 0);
        }
    }
    return true;
}

// ------------------------------------------------------------------ the kernel
// GATHER selects how the A operand reaches shared memory:
//   0  TMA loads through tmapA (every product of a linear layer, and the conv's materialised im2col matrix);
//   1  conv forward: A = the im2col matrix, rows = output pixels (MN-major in shared memory), gathered from the
//      NCHW input by four extra warps; the matrix never exists in global memory;
//   2  conv dW: A = the transposed im2col matrix, rows = k, reduction over pixels (K-major), gathered likewise.
// The gather warps come after the B producer warp; warp 0 then has nothing to do.  They work as two groups of two
// warps that take alternate stages, so two stages are being filled at any time and each thread keeps six 16-byte
// loads in flight; a stage's `full` barrier counts the B producer plus the two warps of the group that fills it.
constexpr int GATHER_WARPS = 8, GATHER_GROUPS = 4;
static_assert(GATHER_GROUPS == STAGES, "each gather group owns one ring slot");

template <bool A_MN, bool B_MN, int GATHER = 0>
__global__ void __launch_bounds__(GATHER ? GATHER_THREADS : GEMM_MAX_THREADS, 1)
sparsedrop_gemm_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                       const __grid_constant__ CUtensorMap tmapC, const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t tiles = (raw_addr + 1023u) & ~1023u;   // 128B swizzle atoms need 1024-byte alignment
    uint8_t* aligned = smem_raw + (tiles - raw_addr);
    uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + TILE_SMEM + STAGING_BYTES);
    // bars[0..3] full, [4..7] empty, [8..9] tmem_full, [10..11] tmem_empty, [12] unused
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 14);
    uint8_t* staging = aligned + TILE_SMEM;   // 32 KiB of TMA-store staging, 1024-aligned
    int4* tab = reinterpret_cast<int4*>(aligned + TILE_SMEM + STAGING_BYTES + 256);   // tile table, TAB_BYTES

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_warps = blockDim.x >> 5;
    const int b_producer_warp = n_warps - 1 - (GATHER ? GATHER_WARPS : 0);
    const int epi_warps = n_warps - 3 - (GATHER ? GATHER_WARPS : 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, GATHER ? 3 : 2);            // the A producer (or two gather warps) and the B producer
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, epi_warps);               // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_mbar_init();
        if (!GATHER) tma_prefetch_desc(&tmapA);
        tma_prefetch_desc(&tmapB);
        if (g.tma_store) tma_prefetch_desc(&tmapC);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched only this CTA's own resources, so it may overlap the tail of the previous kernel in
    // the stream; everything below reads operands, plan lists or workspace that kernel may have produced.
    grid_dep_launch();
    grid_dep_wait();

    const int n_ctas = gridDim.x, cta = blockIdx.x;
    if (g.use_table) {
        WorkIter it;
        it.init(g, cta, n_ctas, tab);
        if (it.tab) {                            // same decision in every thread and, below, in every role
            it.fill_table(g, tab, threadIdx.x, blockDim.x);
            __syncthreads();
        }
    }

    if (warp == 0 || warp == b_producer_warp) {
        // ============================== producers: warp 0 loads the A tiles, the last warp the B tiles.  Two threads
        // because one thread issues a tensor load only every ~110 cycles: the six loads of a stage with both operands
        // MN-major, or the index walk between the short tiles of a conv, would otherwise sit on the critical path.
        // Each arrives on the stage's `full` barrier with its own byte count.
        const bool loads_a = warp == 0;
        if (lane == 0 && !(GATHER && loads_a)) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            WorkIter it;
            it.init(g, cta, n_ctas, tab);
            Seg w;
            while (ok && it.next(g, w)) {
                const uint32_t tx = loads_a ? A_BYTES : (w.b_row1 >= 0 ? B_BYTES : B_HALF_BYTES);
                KIter kit;
                kit.init(w);
                int kb;
                while (ok && kit.next(kb)) {
                    for (int h = 0; h < 2; ++h) {
                        const int k = kb * 128 + h * BK;
                        if (k >= g.KK) break;
                        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, g.status, ST_PRODUCER)) { ok = false; break; }
                        const uint32_t full = bar_full + 8 * stage;
                        mbar_arrive_expect_tx(full, tx);
                        const uint32_t sA = tiles + stage * STAGE_BYTES, sB = sA + A_BYTES;
                        if (loads_a) {
                            if (g.a_panel_kg) {
                                // panels: the 128 pixels of a block are one panel's columns, its k-rows consecutive rows
                                if (!A_MN) {                     // A = colT, rows = k, reduction over pixels
                                    tma_load_2d(sA, &tmapA, full, k & 127, (k >> 7) * g.a_panel_kg + w.a_row);
                                } else {                         // A = col, rows = pixels, reduction over k
                                    const int y = (w.a_row >> 7) * g.a_panel_kg + k;
                                    tma_load_2d(sA, &tmapA, full, 0, y);
                                    tma_load_2d(sA + MN_ATOM_BYTES, &tmapA, full, 64, y);
                                }
                            } else if (!A_MN) {
                                tma_load_2d(sA, &tmapA, full, k, w.a_row);
                            } else {
                                tma_load_2d(sA, &tmapA, full, w.a_row, k);
                                tma_load_2d(sA + MN_ATOM_BYTES, &tmapA, full, w.a_row + 64, k);
                            }
                        } else if (!B_MN) {
                            tma_load_2d(sB, &tmapB, full, k, w.b_row0);
                            if (w.b_row1 >= 0) tma_load_2d(sB + B_HALF_BYTES, &tmapB, full, k, w.b_row1);
                        } else {
                            tma_load_2d(sB, &tmapB, full, w.b_row0, k);
                            tma_load_2d(sB + MN_ATOM_BYTES, &tmapB, full, w.b_row0 + 64, k);
                            if (w.b_row1 >= 0) {
                                tma_load_2d(sB + 2 * MN_ATOM_BYTES, &tmapB, full, w.b_row1, k);
                                tma_load_2d(sB + 3 * MN_ATOM_BYTES, &tmapB, full, w.b_row1 + 64, k);
                            }
                        }
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ============================== MMA issuer
        // The whole warp runs the loops below (every lane sees the same values, so the compiler may keep them in
        // uniform registers, which is where tcgen05.mma takes its descriptors from); one elected lane issues.  Measured
        // against a lone thread inside an `if (lane == 0)`: 2 % faster at 4096^3.
        {
            constexpr uint64_t A_HI = A_MN ? make_smem_desc_hi(MN_ATOM_BYTES, 1024) : make_smem_desc_hi(16, 1024);
            constexpr uint64_t B_HI = B_MN ? make_smem_desc_hi(MN_ATOM_BYTES, 1024) : make_smem_desc_hi(16, 1024);
            constexpr uint32_t A_KSTEP = A_MN ? 2048 : 32;   // bytes per 16-wide K step
            constexpr uint32_t B_KSTEP = B_MN ? 2048 : 32;
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            WorkIter it;
            it.init(g, cta, n_ctas, tab);
            Seg w;
            for (int seg = 0; ok && it.next(g, w); ++seg) {
                if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, g.status, ST_MMA_ACC)) break;
                uint32_t accumulate = 0;
                tc_fence_after();
                const uint32_t d = tmem_base + acc * BN;
                const uint32_t idesc = w.b_row1 >= 0 ? g.idesc256 : g.idesc128;
                // The issuer needs no K coordinates, only how many stages the producers will fill for this segment: two
                // per K tile, one for the last K tile of the matrix when that is at most 64 wide.  The loop below holds
                // nothing but the wait, the four MMAs and the commit: on short tiles (a few stages each) whatever else
                // the issuer does per stage shows up as idle tensor-pipe time.
                int n_stages = 2 * (w.i1 - w.i0);
                if (n_stages > 0 && ((g.KK - 1) & 127) < BK) {
                    const int last = w.use_bits ? 31 - __clz(w.bits) : (w.klist ? __ldg(w.klist + w.i1 - 1) : w.i1 - 1);
                    if (last == ((g.KK + 127) >> 7) - 1) --n_stages;
                }
                for (int st = 0; st < n_stages; ++st) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status, ST_MMA_FULL)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sA = tiles + stage * STAGE_BYTES, sB = sA + A_BYTES;
                    if (elect_one()) {
#pragma unroll
                        for (int j = 0; j < BK / 16; ++j) {
                            umma_f16(d, make_smem_desc(sA + j * A_KSTEP, A_HI), make_smem_desc(sB + j * B_KSTEP, B_HI),
                                     idesc, accumulate);
                            accumulate = 1;
                        }
                        umma_commit(bar_empty + 8 * stage);
                    }
                    accumulate = 1;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (elect_one()) umma_commit(bar_tfull + 8 * acc);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
        __syncwarp();
    } else if (GATHER && warp > b_producer_warp) {
        // ============================== gather warps: build the A tile of a stage from the NCHW input.
        // One work item = one aligned 8-pixel chunk of one input row for one (channel, filter row): the three taps
        // s = 0, 1, 2 are that chunk shifted by -1, 0, +1 pixel, the pixel that comes in at either end is traded
        // with the neighbouring lane (which owns the neighbouring chunk of the same image row), and the item writes
        // up to three k-rows of the 128B-swizzled stage.  Rows and pixels that do not exist are written as zeros.
        // Group j (two warps) fills ring slot j.  The loads of a group's next stage are issued before its current
        // stage is stored, so their latency hides behind the stores and the wait for the slot; loads and stores are
        // predicated, not branched around, and each helper below is expanded exactly once.
        const int gw = warp - b_producer_warp - 1, group = gw >> 1;   // group == ring slot (GATHER_GROUPS == STAGES)
        const int t = ((gw & 1) << 5) | lane;                         // 0..63 inside the group
        const ConvGather& cv = g.conv;
        // GATHER 1: 16 pixel chunks x 4 (c, r) pairs per pass;  GATHER 2: 8 pixel chunks x 8 pairs per pass
        const int chunk = GATHER == 1 ? (t & 15) : (t & 7), tsub = GATHER == 1 ? (t >> 4) : (t >> 3);
        constexpr int PAIRS_PER_PASS = GATHER == 1 ? 4 : 8, PASSES = 6, STAGE_ROWS = GATHER == 1 ? BK : 128;
        const uint32_t piece = GATHER == 1 ? (chunk & 7) : chunk;
        const uint32_t slot_base = tiles + group * STAGE_BYTES + (GATHER == 1 ? uint32_t(chunk >> 3) * MN_ATOM_BYTES : 0u);
        const uint32_t slot_full = bar_full + 8 * group, slot_empty = bar_empty + 8 * group;

        struct StageJob {
            uint32_t parity;       // parity to wait for on the slot's `empty` barrier
            int k_lo, rows;        // first k-row of the im2col matrix in the stage, and how many exist
            int cr0, cr_end;       // this thread's first (channel, filter row) pair, and the end of the stage's pairs
            bool has_left, has_right;
        };
        // Walks the CTA's stages in the order every role sees them and stops at those of this group's slot.
        WorkIter it;
        it.init(g, cta, n_ctas, tab);
        Seg w;
        KIter kit;
        int kb = 0, h = 2, ring = 0;
        uint32_t phase = 0;
        bool in_tile = false;
        const unsigned short* xrow = cv.x;      // this thread's 8 pixels in channel 0, input row 0 (may lie outside the image)
        int hbase = 0;
        bool live = false, has_left = false, has_right = false;
        auto decode_pixels = [&](int m0) {      // m0: first of this thread's 8 consecutive output pixels
            live = m0 < cv.pixels;
            const int mm = live ? m0 : 0;
            const int n = fast_div(mm, cv.mul_pq, cv.shr_pq), pq = mm - n * cv.PQ;
            const int pp = pq >> cv.log2_w, q0 = pq & (cv.W - 1);
            xrow = cv.x + (long long)n * cv.C * cv.HW + q0;
            hbase = pp * cv.stride_h - cv.pad_h;
            has_left = q0 > 0;
            has_right = q0 + 8 < cv.W;
        };
        auto next_job = [&](StageJob& job) -> bool {
            for (;;) {
                if (!in_tile) {
                    if (!it.next(g, w)) return false;
                    in_tile = true;
                    kit.init(w);
                    h = 2;
                    if (GATHER == 1) decode_pixels(w.a_row + chunk * 8);         // pixels are the tile's rows
                }
                if (h == 2) {                                                    // next K tile of the segment
                    if (!kit.next(kb)) { in_tile = false; continue; }
                    h = 0;
                }
                const int k = kb * 128 + h * BK;
                if (k >= g.KK) { h = 2; continue; }
                ++h;
                const bool mine = ring == group;
                job.parity = phase ^ 1;
                if (++ring == STAGES) { ring = 0; phase ^= 1; }
                if (!mine) continue;
                job.k_lo = GATHER == 1 ? k : w.a_row;
                const int k_hi = min(job.k_lo + STAGE_ROWS, cv.k_real);
                job.rows = k_hi - job.k_lo;
                job.cr0 = job.k_lo / 3 + tsub;
                job.cr_end = (k_hi + 2) / 3;
                if (GATHER == 2) decode_pixels(k + chunk * 8);                   // pixels are the reduction index
                job.has_left = has_left;
                job.has_right = has_right;
                return true;
            }
        };
        auto issue_loads = [&](const StageJob& job, uint4 (&v)[PASSES]) {
            int c = fast_div(job.cr0, cv.mul_r, cv.shr_r), r = job.cr0 - c * cv.R;
#pragma unroll
            for (int u = 0; u < PASSES; ++u) {
                const int hh = hbase + r * cv.dil_h;
                const bool pred = live && job.cr0 + PAIRS_PER_PASS * u < job.cr_end && (unsigned)hh < (unsigned)cv.H;
                v[u] = ldg_nc_v4_pred(xrow + (long long)c * cv.HW + hh * cv.W, pred);
                c += cv.pass_dc[GATHER];                                  // (c, r) of the pair PAIRS_PER_PASS further on
                r += cv.pass_dr[GATHER];
                if (r >= cv.R) { r -= cv.R; ++c; }
            }
        };
        // Stores the stage.  Returns false if the wait for the slot was abandoned.
        auto store_stage = [&](const StageJob& job, const uint4 (&v)[PASSES]) -> bool {
            bool ok = mbar_wait(slot_empty, job.parity, abort_flag, g.status, ST_PRODUCER);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return false;
            // address of (k-row kk, this thread's chunk): MN-major stage = two 64-pixel atoms of 64 k-rows of 128
            // bytes; K-major stage = 128 k-rows of 128 bytes; 16-byte pieces XOR-swizzled by the row
            auto put = [&](int kk, bool pred, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
                st_shared_v4_pred(slot_base + uint32_t(kk) * 128u + ((piece ^ (uint32_t(kk) & 7u)) << 4), pred, a, b, c, d);
            };
#pragma unroll
            for (int u = 0; u < PASSES; ++u) {
                const int cr = job.cr0 + PAIRS_PER_PASS * u;
                uint32_t left = __shfl_up_sync(0xffffffffu, v[u].w, 1);
                uint32_t right = __shfl_down_sync(0xffffffffu, v[u].x, 1);
                if (!job.has_left) left = 0;
                if (!job.has_right) right = 0;
                const bool on = cr < job.cr_end;
                const int kk = 3 * cr - job.k_lo;                // stage row of tap s = 0; -2 .. rows - 1
                const uint32_t a0 = __funnelshift_r(v[u].x, v[u].y, 16), a1 = __funnelshift_r(v[u].y, v[u].z, 16),
                               a2 = __funnelshift_r(v[u].z, v[u].w, 16);
                put(kk, on && kk >= 0, __funnelshift_r(left, v[u].x, 16), a0, a1, a2);
                put(kk + 1, on && kk + 1 >= 0 && kk + 1 < job.rows, v[u].x, v[u].y, v[u].z, v[u].w);
                put(kk + 2, on && kk + 2 < job.rows, a0, a1, a2, __funnelshift_r(v[u].w, right, 16));
            }
            // k-rows past the end of the im2col matrix multiply zero-filled B rows: they must be zeros, not
            // whatever the stage held before
            for (int kk = job.rows + tsub; kk < STAGE_ROWS; kk += PAIRS_PER_PASS) put(kk, true, 0, 0, 0, 0);
            fence_proxy_async();                                 // generic-proxy writes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(slot_full);
            return true;
        };
        StageJob cur, nxt;
        uint4 vc[PASSES], vn[PASSES];
        bool have_cur = false;
        for (;;) {
            const bool have_nxt = next_job(nxt);
            if (have_nxt) issue_loads(nxt, vn);
            if (have_cur && !store_stage(cur, vc)) break;
            if (!have_nxt) break;
            cur = nxt;
#pragma unroll
            for (int u = 0; u < PASSES; ++u) vc[u] = vn[u];
            have_cur = true;
        }
        __syncwarp();
    } else {
        // ============================== epilogue
        // Warps 2..5 and 6..9 own TMEM lane quadrants 2,3,0,1 (a warp reaches only the 32 lanes of quadrant warp % 4);
        // the first four take the lower half of a tile's column chunks, the other four the upper half.
        const int epi_halves = epi_warps >> 2, epi_threads = epi_warps << 5;
        const bool two_bufs = epi_warps == 4;
        const int quad = warp & 3, half = (warp - 2) >> 2;       // half is 0 throughout with four epilogue warps
        const int etid = quad * 32 + lane;   // 0..127, also the row inside the tile this thread owns
        const int eidx = half * 128 + etid;  // 0..255, index inside the epilogue group
        const bool aligned16 = (reinterpret_cast<uintptr_t>(g.C) & 15) == 0;
        const bool vec_ok = g.c_cs == 1 && (g.c_rs & 7) == 0 && aligned16;      // row-major result, 16-byte rows
        const bool vec_t_ok = g.c_rs == 1 && (g.c_cs & 7) == 0 && aligned16;    // column-major result
        // Output that no unit covers is zero-filled here, before the first accumulator is ready.
        if (g.mode == MODE_SDD && g.n_zero) {
            const int nz = __ldg(g.n_zero);
            for (int z = epi_halves * cta + half; z < nz; z += epi_halves * n_ctas)
                zero_tile(g, vec_ok, vec_t_ok, etid, __ldg(g.zero_pairs + 2 * z) * 128, __ldg(g.zero_pairs + 2 * z + 1) * 128);
        } else if (g.mode == MODE_DSD) {
            // row blocks with nothing kept: their 128x128 output tiles are spread over all CTAs
            // Every warp of the group tests the same 32 candidates at a time, one per lane, so the index loads of a
            // whole batch are in flight together; the ballot then gives all of them the same list of tiles to zero.
            const int ncol = (g.NN + 127) >> 7, total = g.n_row_blocks * ncol;
            const int z0 = epi_halves * cta + half, zstep = epi_halves * n_ctas;
            for (int zb = z0; zb < total; zb += 32 * zstep) {
                const int z = zb + lane * zstep;
                bool empty = false;
                if (z < total) {
                    const int rb = z / ncol;
                    empty = __ldg(g.list_ptr + rb + 1) == __ldg(g.list_ptr + rb);
                }
                unsigned found = __ballot_sync(0xffffffffu, empty);
                while (found) {
                    const int zz = zb + (__ffs(found) - 1) * zstep, rb = zz / ncol;
                    found &= found - 1;
                    zero_tile(g, vec_ok, vec_t_ok, etid, rb * 128, (zz - rb * ncol) * 128);
                }
            }
        }
        WorkIter it;
        it.init(g, cta, n_ctas, tab);
        int acc = 0;
        uint32_t acc_phase = 0;
        Seg w;
        // Split schedule: the tile this CTA shares with the rest of its group; reduced after the segment loop.
        Seg shared;
        bool has_shared = false;
        const uint32_t stage_base = smem_u32(staging) + uint32_t(warp - 2) * (two_bufs ? 8192u : 4096u);   // this warp's staging
        int n_stores = 0;
        bool alive = true;
        while (alive && it.next(g, w)) {
            const bool partial = w.parts > 1;
            const bool ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, g.status, ST_EPILOGUE);
            // Split launches synchronise all epilogue warps later (the shared tile), so they decide together whether
            // to go on; otherwise every warp decides for itself and no warp waits for the slowest one at every tile.
            if (g.split ? !epilogue_all(ok, epi_threads) : !__all_sync(0xffffffffu, ok)) { alive = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + acc * BN + (uint32_t(quad * 32) << 16);
            const int row = w.a_row + etid;
            const int nchunks = (w.b_row1 >= 0 ? 8 : 4) >> (epi_halves - 1);   // this warp's share: chunks [c0, c0 + nchunks)
            const int c0 = half * nchunks;
            float* slot = nullptr;
            if (partial) slot = g.ws_slots + size_t(cta) * WS_SLOT_FLOATS;
            // One chunk: 32 rows x 32 fp32 columns in r, thread = row.  `odd` chunks close a pair.
            // Elementwise work on a chunk before it is converted: the fused ReLU, or the mask of a ReLU's derivative.
            auto fix = [&](const int c, uint32_t (&r)[32]) {
                if (partial) return;                             // shared tiles are finished by reduce_shared_tile
                if (g.act == 1) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = int(r[j]) < 0 ? 0u : r[j];   // sign bit set -> 0
                }
                if (g.mask_src) {
                    const int col = c < 4 ? w.b_row0 + c * 32 : w.b_row1 + (c - 4) * 32;
                    if (row < g.MM) {
                        const uint4* src = reinterpret_cast<const uint4*>(g.mask_src + (long long)row * g.mask_rs + col);
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            if (col + 8 * v >= g.NN) break;      // N is a multiple of 8 here: whole groups in or out
                            const uint4 q = __ldg(src + v);
                            const uint32_t wv[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (short(wv[j] & 0xffffu) <= 0) r[8 * v + 2 * j] = 0u;
                                if (short(wv[j] >> 16) <= 0) r[8 * v + 2 * j + 1] = 0u;
                            }
                        }
                    }
                }
            };
            auto process = [&](const int c, const uint32_t (&r)[32]) {
                const int col = c < 4 ? w.b_row0 + c * 32 : w.b_row1 + (c - 4) * 32;
                if (partial) {
                    // unit (chunk c, quadrant) = 32 rows x 32 fp32 columns stored as [4-column piece][row]: each warp
                    // store instruction writes 512 contiguous bytes
                    uint4* dst = reinterpret_cast<uint4*>(slot + size_t(c * 4 + quad) * 1024) + lane;
#pragma unroll
                    for (int v = 0; v < 8; ++v) __stcg(dst + v * 32, make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]));
                } else if (g.tma_store == 1) {
                    // Two chunks (32 rows x 64 columns) share the 4 KiB staging buffer of 128-byte rows, 16-byte pieces
                    // XOR-swizzled as CU_TENSOR_MAP_SWIZZLE_128B expects, and leave by one TMA store: the proxy fence and
                    // the store's issue cost a few hundred cycles, so they are paid once per pair.
                    const uint32_t buf = stage_base + (two_bufs ? ((n_stores & 1) << 12) : 0);
                    if (!(c & 1)) wait_staging_free(two_bufs, n_stores, lane);
                    const uint32_t rowaddr = buf + lane * 128, sw = lane & 7, piece0 = (c & 1) << 2;
                    uint32_t p[16];
                    convert_chunk(r, g.scale, g.is_bf16, p);
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (((piece0 + v) ^ sw) << 4)),
                                     "r"(p[4 * v]), "r"(p[4 * v + 1]), "r"(p[4 * v + 2]), "r"(p[4 * v + 3])
                                     : "memory");
                    if (c & 1) {
                        fence_proxy_async();
                                                __syncwarp();
                        if (lane == 0) {
                            if (!g.c_panel_kg)
                                tma_store_2d(&tmapC, buf, col - 32, w.a_row + quad * 32);
                            else if (w.a_row + quad * 32 < g.MM) { // rows past the last k would land in the next panel
                                const int pix0 = c < 4 ? w.b_row0 : w.b_row1;     // the pixel block of this half
                                tma_store_2d(&tmapC, buf, col - 32 - pix0,
                                             (pix0 >> 7) * g.c_panel_kg + w.a_row + quad * 32);
                            }
                            bulk_commit();
                        }
                        ++n_stores;
                                            }
                } else if (g.tma_store == 2) {
                    // column-major result = row-major transpose: the warp's 32 rows x 64 columns are staged as
                    // [column][row] (64-byte rows of the transpose, CU_TENSOR_MAP_SWIZZLE_64B) and stored by one TMA store
                    const uint32_t buf = stage_base + (two_bufs ? ((n_stores & 1) << 12) : 0);
                    if (!(c & 1)) wait_staging_free(two_bufs, n_stores, lane);
                    const uint32_t hbuf = buf + ((c & 1) << 11), lane_off = ((lane & 7) << 1), chunk = lane >> 3;
                    uint32_t p[16];
                    convert_chunk(r, g.scale, g.is_bf16, p);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t addr = hbuf + j * 64 + (((chunk ^ ((j >> 1) & 3))) << 4) + lane_off;
                        asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"((unsigned short)(p[j >> 1] >> (16 * (j & 1))))
                                     : "memory");
                    }
                    if (c & 1) {
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d(&tmapC, buf, w.a_row + quad * 32, col - 32);
                            bulk_commit();
                        }
                        ++n_stores;
                    }
                } else if (g.tma_store == 3) {
                    // fp32 column-major result (a weight gradient written into the fp32 gradient buffer): one chunk =
                    // 32 columns of 32 rows = 4 KiB, staged as [column][row] (128-byte rows of the transpose,
                    // CU_TENSOR_MAP_SWIZZLE_128B) and stored by one TMA store
                    const uint32_t buf = stage_base + (two_bufs ? ((n_stores & 1) << 12) : 0);
                    wait_staging_free(two_bufs, n_stores, lane);
                    const uint32_t piece = uint32_t(lane) >> 2, within = (uint32_t(lane) & 3u) << 2;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t addr = buf + j * 128 + ((piece ^ (uint32_t(j) & 7u)) << 4) + within;
                        asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "f"(__uint_as_float(r[j]) * g.scale) : "memory");
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tmapC, buf, w.a_row + quad * 32, col);
                        bulk_commit();
                    }
                    ++n_stores;
                } else if (g.out_f32) {
                    store_chunk_f32(g, row, col, r);
                } else {
                    store_chunk(g, vec_ok, row, col, r);
                }
            };
            // chunk c+1 is in flight from TMEM while chunk c is converted and stored; chunks come in pairs (c0 and the
            // chunk count are even), even ones through rbuf[0] and odd ones through rbuf[1]
            uint32_t rbuf[2][32];
            tmem_ld_32x32(taddr + c0 * 32, rbuf[0]);
            tmem_ld_wait();
            for (int c = c0; c < c0 + nchunks; c += 2) {
                tmem_ld_32x32(taddr + (c + 1) * 32, rbuf[1]);
                if (g.act | (g.mask_src != nullptr)) fix(c, rbuf[0]);
                process(c, rbuf[0]);
                tmem_ld_wait();
                if (g.act | (g.mask_src != nullptr)) fix(c + 1, rbuf[1]);
                if (c + 2 < c0 + nchunks) tmem_ld_32x32(taddr + (c + 2) * 32, rbuf[0]);
                process(c + 1, rbuf[1]);
                tmem_ld_wait();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
            if (partial) {
                __threadfence();                                 // partial tile visible before the arrival count
                epilogue_sync(epi_threads);
                if (eidx == 0) atomicAdd(g.ws_flags + w.owner, 1);
                shared = w;
                has_shared = true;
            }
        }
        if (g.tma_store && lane == 0) bulk_wait_all();           // staged results are in global memory
        __syncwarp();
        if (alive && has_shared) alive = reduce_shared_tile(g, shared, eidx, epi_threads, abort_flag);
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Tensor map of one 16-bit operand X[rows, kk] given its two element strides.
//   column stride 1 -> K-major : global (kk, rows),  box 64 x 128
//   row stride 1    -> MN-major: global (rows, kk),  box 64 x 64
static int make_operand_map(CUtensorMap* out, bool* mn_major, const char* name, const void* ptr, int64_t rs, int64_t cs,
                            int rows, int kk, int dtype) {
    if (!ptr) return fail(SD_ERR_INVALID_ARG, "%s is null", name);
    const bool k_major = (cs == 1);
    if (!k_major && rs != 1) return fail(SD_ERR_LAYOUT, "%s must be row or column major", name);
    const int64_t ld = k_major ? rs : cs;
    const int64_t inner = k_major ? kk : rows, outer = k_major ? rows : kk;
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(SD_ERR_LAYOUT, "%s must be 16-byte aligned", name);
    if (outer > 1 && (ld < inner || (ld & 7)))
        return fail(SD_ERR_LAYOUT, "%s leading stride (%lld) must be >= %lld and a multiple of 8 elements", name,
                    (long long)ld, (long long)inner);
    // Bind the device's primary context to this thread before the first driver-API call: a thread that has
    // made no runtime call yet (e.g. an autograd worker) has no current context and cuTensorMapEncodeTiled
    // would fail with CUDA_ERROR_INVALID_CONTEXT.  Done once per thread and device.
    int dev = 0;
    SD_CUDA_TRY(cudaGetDevice(&dev));
    static thread_local int bound_device = -1;
    if (bound_device != dev) {
        SD_CUDA_TRY(cudaSetDevice(dev));
        bound_device = dev;
    }
    // Small per-thread cache: training loops present the same few operands over and over.
    struct MapKey {
        const void* ptr; int64_t ld; int rows, kk, dtype, dev; bool k_major;
        bool operator==(const MapKey& o) const {
            return ptr == o.ptr && ld == o.ld && rows == o.rows && kk == o.kk && dtype == o.dtype && dev == o.dev &&
                   k_major == o.k_major;
        }
    };
    constexpr int kCache = 32;
    static thread_local MapKey keys[kCache];
    static thread_local CUtensorMap maps[kCache];
    static thread_local int used = 0, next_slot = 0;
    const MapKey key{ptr, ld, rows, kk, dtype, dev, k_major};
    for (int i = 0; i < used; ++i)
        if (keys[i] == key) {
            *out = maps[i];
            *mn_major = !k_major;
            return SD_OK;
        }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(SD_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable in this driver");
    cuuint64_t dims[2] = {cuuint64_t(inner), cuuint64_t(outer)};
    cuuint64_t strides[1] = {cuuint64_t(outer > 1 ? ld * 2 : ((inner * 2 + 15) & ~int64_t(15)))};
    cuuint32_t box[2] = {64u, k_major ? 128u : 64u};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = enc(out, dtype == SD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                     const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SD_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", name, int(r));
    const int slot = used < kCache ? used++ : (next_slot = (next_slot + 1) % kCache);
    keys[slot] = key;
    maps[slot] = *out;
    *mn_major = !k_major;
    return SD_OK;
}

template <bool A_MN, bool B_MN, int GATHER = 0>
static int launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmArgs& g, int grid,
                          int epi_warps, cudaStream_t st) {
    // Called from the main thread and from autograd's worker threads at once: the per-device "already configured"
    // flags are atomics (setting the attribute twice is harmless, so relaxed ordering is enough).
    static std::atomic<bool> configured[64] = {};
    int dev = 0;
    SD_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev].load(std::memory_order_relaxed)) {
        SD_CUDA_TRY(cudaFuncSetAttribute(sparsedrop_gemm_kernel<A_MN, B_MN, GATHER>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM));
        if (dev < 64) configured[dev].store(true, std::memory_order_relaxed);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(96 + 32 * epi_warps + (GATHER ? 32 * GATHER_WARPS : 0));
    cfg.dynamicSmemBytes = GEMM_SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // prologue may overlap the previous kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    SD_CUDA_TRY(cudaLaunchKernelEx(&cfg, sparsedrop_gemm_kernel<A_MN, B_MN, GATHER>, ta, tb, tc, g));
    return SD_OK;
}

// SMs that the persistent grids of this library leave free (sd_set_sm_margin); SD_SM_MARGIN gives the initial value.
static std::atomic<int> g_sm_margin{[] {
    const char* e = getenv("SD_SM_MARGIN");
    const int v = e ? atoi(e) : 0;
    return v > 0 ? v : 0;
}()};

// Optional epilogue work of one launch (see the fields of the same names in GemmArgs).
struct GemmExtras {
    int act = 0;
    const void* mask_src = nullptr;
    int64_t mask_rs = 0;
    int out_f32 = 0, out_acc = 0;
};

struct PlanView {
    const int *header, *row_ptr, *col_idx, *col_ptr, *row_idx, *row_order, *col_order, *sdd_items, *drop_pairs, *kept_pairs;
    const unsigned char* mask;
};
static PlanView view_plan(const void* plan, int R, int C) {
    const sd_plan_layout L = plan_layout(R, C);
    const unsigned char* b = static_cast<const unsigned char*>(plan);
    PlanView v;
    v.header = reinterpret_cast<const int*>(b + L.header);
    v.row_ptr = reinterpret_cast<const int*>(b + L.row_ptr);
    v.col_idx = reinterpret_cast<const int*>(b + L.col_idx);
    v.col_ptr = reinterpret_cast<const int*>(b + L.col_ptr);
    v.row_idx = reinterpret_cast<const int*>(b + L.row_idx);
    v.row_order = reinterpret_cast<const int*>(b + L.row_order);
    v.col_order = reinterpret_cast<const int*>(b + L.col_order);
    v.sdd_items = reinterpret_cast<const int*>(b + L.sdd_items);
    v.drop_pairs = reinterpret_cast<const int*>(b + L.drop_pairs);
    v.kept_pairs = reinterpret_cast<const int*>(b + L.kept_pairs);
    v.mask = b + L.mask;
    return v;
}

static int run_gemm(int mode, const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs,
                    void* C, int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, int plan_side,
                    float scale, int dtype, void* workspace, int* status, void* stream, int max_ctas = 0,
                    bool zero_dropped = true, bool sdd_t = false, int panels = 0, const ConvGather* conv = nullptr,
                    int gather = 0, const GemmExtras* extras = nullptr) {
    // gather: 1 / 2 = A is the im2col matrix of `conv` (rows = pixels) / its transpose (rows = k), built inside the
    // kernel from the NCHW input; A, a_rs, a_cs are then ignored.
    // panels: 1 = A is the conv's im2col matrix in panels of 128 pixels ([pixels/128][kg][128]); DSD with the plan's
    // rows = pixel blocks: side ROWS means A[M = pixels, K = kg], side COLS means A[M = kg, K = pixels].
    // 2 = C[M = kg, N = pixels] is stored that way (SDD for the transposed plan).  kg must be a multiple of 64.
    if (M <= 0 || N <= 0 || K <= 0) return fail(SD_ERR_INVALID_ARG, "M, N, K must be positive (got %d, %d, %d)", M, N, K);
    if (dtype != SD_F16 && dtype != SD_BF16) return fail(SD_ERR_INVALID_ARG, "dtype must be SD_F16 or SD_BF16");
    if (!C) return fail(SD_ERR_INVALID_ARG, "C is null");
    if (c_rs != 1 && c_cs != 1) return fail(SD_ERR_LAYOUT, "C must be row or column major");
    if (mode != MODE_DENSE && !plan) return fail(SD_ERR_INVALID_ARG, "plan is null");
    if (mode == MODE_DSD && plan_side != SD_PLAN_ROWS && plan_side != SD_PLAN_COLS)
        return fail(SD_ERR_INVALID_ARG, "plan_side must be SD_PLAN_ROWS or SD_PLAN_COLS");

    if (panels == 2 && (M & 63))
        return fail(SD_ERR_LAYOUT, "panel layout needs a k extent that is a multiple of 64 (got %d)", M);
    CUtensorMap ta, tb;
    bool a_mn = false, b_mn = false;
    int rc;
    int a_panel_kg = 0, c_panel_kg = 0;
    if (gather) {
        a_mn = gather == 1;
        rc = SD_OK;
    } else if (panels == 1) {
        const bool rows_are_pixels = plan_side == SD_PLAN_ROWS;
        const int pixels = rows_are_pixels ? M : K, kg = rows_are_pixels ? K : M;
        if (kg & 63) return fail(SD_ERR_LAYOUT, "panel layout needs a k extent that is a multiple of 64 (got %d)", kg);
        const long long all_rows = (long long)((pixels + 127) / 128) * kg;
        if (all_rows > (1ll << 31) - 1) return fail(SD_ERR_TOO_LARGE, "panel matrix too large");
        // the panels form one row-major [panels * kg][128] matrix; as an operand: 128 "MN" columns x all_rows, MN-major
        // (boxes of 64 x 64), or all_rows x 128, K-major (boxes of 64 x 128)
        rc = rows_are_pixels ? make_operand_map(&ta, &a_mn, "A", A, 1, 128, 128, int(all_rows), dtype)
                             : make_operand_map(&ta, &a_mn, "A", A, 128, 1, int(all_rows), 128, dtype);
        a_panel_kg = kg;
    } else {
        rc = make_operand_map(&ta, &a_mn, "A", A, a_rs, a_cs, M, K, dtype);
    }
    if (rc) return rc;
    if (panels == 2) {
        if (reinterpret_cast<uintptr_t>(C) & 15) return fail(SD_ERR_LAYOUT, "C must be 16-byte aligned");
        c_panel_kg = M;
        c_rs = 128; c_cs = 1;    // only the TMA path below writes C
    }
    rc = make_operand_map(&tb, &b_mn, "B", B, b_rs, b_cs, N, K, dtype);
    if (rc) return rc;
    if (gather) ta = tb;                       // the kernel never touches tmapA

    GemmArgs g{};
    if (conv) g.conv = *conv;
    if (extras) {
        if (extras->mask_src) {
            if ((reinterpret_cast<uintptr_t>(extras->mask_src) & 15) || (extras->mask_rs & 7) || extras->mask_rs < N || (N & 7))
                return fail(SD_ERR_LAYOUT, "the mask source must be row-major with 16-byte aligned rows (N and its row "
                                           "stride multiples of 8, got N=%d, stride %lld)", N, (long long)extras->mask_rs);
            if (panels || sdd_t) return fail(SD_ERR_INVALID_ARG, "the mask source is not supported for panel or transposed results");
        }
        g.act = extras->act;
        g.mask_src = static_cast<const unsigned short*>(extras->mask_src);
        g.mask_rs = extras->mask_rs;
        g.out_f32 = extras->out_f32;
        g.out_acc = extras->out_acc;
        if (g.out_f32 && (reinterpret_cast<uintptr_t>(C) & 3)) return fail(SD_ERR_LAYOUT, "an fp32 result must be 4-byte aligned");
    }
    g.mode = mode;
    g.MM = M; g.NN = N; g.KK = K;
    g.C = C; g.c_rs = c_rs; g.c_cs = c_cs;
    g.scale = scale;
    g.is_bf16 = dtype == SD_BF16;
    g.n_row_blocks = (M + 127) / 128;
    g.n_col_tiles = (N + BN - 1) / BN;
    g.status = status;
    g.idesc256 = make_idesc(128, 256, g.is_bf16, a_mn, b_mn);
    g.idesc128 = make_idesc(128, 128, g.is_bf16, a_mn, b_mn);
    g.a_panel_kg = a_panel_kg;
    g.c_panel_kg = c_panel_kg;

    int sms = 0;
    rc = sm_count_current_device(&sms);
    if (rc) return rc;
    // SMs left to kernels that run beside this one (a gradient all-reduce overlapping the next step's products): a
    // persistent CTA holds its SM for the whole launch, and with a static deal of tiles a CTA that has to wait for an
    // SM another kernel occupies stretches the launch by up to a whole pass.
    const int sm_margin = g_sm_margin.load(std::memory_order_relaxed);
    int grid = sms > 2 * sm_margin ? sms - sm_margin : sms;
    if (mode == MODE_DSD) {
        const int kb = (K + 127) / 128;
        if (plan_side == SD_PLAN_ROWS) {
            PlanView v = view_plan(plan, g.n_row_blocks, kb);
            g.list_ptr = v.row_ptr; g.list_idx = v.col_idx; g.order = v.row_order;
            g.h_nnz = v.header + H_NNZ; g.h_max = v.header + H_MAX_ROW;
            if (kb <= 32) { g.direct_mask = v.mask; g.dm_stride_rb = kb; g.dm_stride_k = 1; }
        } else {
            PlanView v = view_plan(plan, kb, g.n_row_blocks);
            g.list_ptr = v.col_ptr; g.list_idx = v.row_idx; g.order = v.col_order;
            g.h_nnz = v.header + H_NNZ; g.h_max = v.header + H_MAX_COL;
            if (kb <= 32) { g.direct_mask = v.mask; g.dm_stride_rb = 1; g.dm_stride_k = g.n_row_blocks; }
        }
    } else if (mode == MODE_SDD && sdd_t) {
        // the plan's grid is (N/128) x (M/128): the transpose of the result's; one item per kept pair
        PlanView v = view_plan(plan, (N + 127) / 128, g.n_row_blocks);
        g.items = v.kept_pairs; g.n_items = v.header + H_NNZ;
        g.sdd_single = 2;
        // few result row blocks (the conv's k blocks) with many kept tiles each: pair the tiles of a row block, which
        // halves the number of tiles a CTA walks through and the A traffic
        if (g.n_row_blocks <= 64 && (long long)g.n_row_blocks * ((N + 127) / 128) >= 4ll * sms) {
            g.list_ptr = v.col_ptr; g.list_idx = v.row_idx;
            g.sdd_single = 3;
        }
    } else if (mode == MODE_SDD) {
        PlanView v = view_plan(plan, g.n_row_blocks, (N + 127) / 128);
        // paired items halve the A traffic; with so few of them that half the SMs would idle, one tile per item
        // puts twice as many SMs to work
        const long long pairs_upper = (long long)g.n_row_blocks * ((((N + 127) / 128) + 1) / 2);
        if (pairs_upper * 2 <= sms) {
            g.items = v.kept_pairs; g.n_items = v.header + H_NNZ;
            g.sdd_single = 1;
        } else {
            g.items = v.sdd_items; g.n_items = v.header + H_SDD_ITEMS;
        }
        if (zero_dropped) { g.zero_pairs = v.drop_pairs; g.n_zero = v.header + H_NDROP; }
    }
    // Schedule: with fewer output tiles than SMs, whole tiles would leave SMs idle, so each tile's
    // reduction is split over a group of CTAs instead (needs the workspace).  Otherwise whole tiles, heaviest first.
    const long long tiles_upper = (mode == MODE_SDD && g.sdd_single) ? (long long)g.n_row_blocks * ((N + 127) / 128)
                                  : mode == MODE_SDD        ? (long long)g.n_row_blocks * ((((N + 127) / 128) + 1) / 2)
                                                            : (long long)g.n_row_blocks * g.n_col_tiles;
    if (max_ctas > 0) {
        if (tiles_upper > max_ctas)
            return fail(SD_ERR_TOO_LARGE,
                        "%lld output tiles of 128x256 exceed the %d the built-in scratch serves; launches this large "
                        "need no scratch: call sd_gemm_dsd with workspace = NULL",
                        tiles_upper, max_ctas);
        if (grid > max_ctas) grid = max_ctas;
    }
    // Cutting tiles pays only when each tile is long: the partial-tile exchange costs about as much as a dozen
    // K tiles, so short reductions keep whole tiles even on an under-filled grid.
    const int k_tiles = (K + 127) / 128;
    static const int split_min_k_tiles = [] {
        const char* e = getenv("SD_SPLIT_MIN_KTILES");   // tuning knob: minimum reduction length (in 128-wide K tiles)
        return e ? atoi(e) : 16;
    }();
    const bool elementwise = g.mask_src != nullptr;   // the mask is applied by whole-tile epilogues only
    static const int small_halves = [] {
        const char* e = getenv("SD_SMALL_HALVES");         // tuning knob: 0 keeps whole 128x256 tiles on small launches
        return e ? atoi(e) : 1;
    }();
    if (workspace && tiles_upper * 2 <= grid && k_tiles >= split_min_k_tiles && !c_panel_kg && !elementwise) {
        if (reinterpret_cast<uintptr_t>(workspace) & 15) return fail(SD_ERR_LAYOUT, "workspace must be 16-byte aligned");
        if (grid > WS_MAX_CTAS) grid = WS_MAX_CTAS;
        g.split = 1;
        g.ws_flags = static_cast<int*>(workspace);
        g.ws_slots = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + WS_FLAG_BYTES);
    } else if (small_halves && mode != MODE_SDD && !gather && N > 128 && tiles_upper * 2 <= grid) {
        // a launch this small is bound by how fast one SM can stream a tile's operands: hand every 128x256 tile out as
        // two 128-wide halves, so that twice as many SMs share the stream
        g.all_halves = 1;
        grid = int(tiles_upper * 2);
    } else if (tiles_upper < grid) {
        grid = int(tiles_upper);
    }
    // Whole-tile launches describe their tiles once per CTA in shared memory when a tile's kept K tiles fit a 32-bit mask
    // (and only when a CTA gets enough tiles for the table to pay: see TAB_MIN; the bound below counts every tile
    // that may exist, the kernel checks the tiles that do)
    // Short reductions (up to 16 K tiles) make a tile so short that resolving the next one between tiles shows: they get
    // the table from five passes on ((16384, 1536, 384) forward: 25.3 -> 22.5 us); long ones only from TAB_MIN on, where
    // the table's prologue would otherwise cost more than it saves (4096^3: +2.7 %).
    static const int tab_min_short = [] {
        const char* e = getenv("SD_TAB_MIN_SHORT");        // tuning knob: fewest passes that get the table, short reductions
        return e ? atoi(e) : 5;
    }();
    g.tab_min = k_tiles <= 16 ? tab_min_short : TAB_MIN;
    g.use_table = !g.split && (mode != MODE_DSD || k_tiles <= 32) && tiles_upper >= (long long)g.tab_min * grid / 2;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Row-major result with 16-byte rows: written by TMA (clipped at the ragged edge); otherwise by the warps.
    CUtensorMap tc = ta;
    if (g.out_f32) {
        // an fp32 result that overwrites a column-major matrix with 16-byte aligned columns leaves by TMA; other
        // fp32 results (row-major, accumulating, unaligned) are written by the epilogue warps directly
        if (!g.out_acc && c_rs == 1 && (c_cs & 3) == 0 && c_cs >= M && (reinterpret_cast<uintptr_t>(C) & 15) == 0) {
            EncodeTiledFn enc = encode_tiled_fn();
            cuuint64_t dims[2] = {cuuint64_t(M), cuuint64_t(N)};            // the transpose, row-major [N][M]
            cuuint64_t strides[1] = {cuuint64_t(N > 1 ? c_cs * 4 : ((int64_t(M) * 4 + 15) & ~int64_t(15)))};
            cuuint32_t box[2] = {32u, 32u};
            cuuint32_t estr[2] = {1u, 1u};
            CUresult r = enc(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, C, dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(SD_ERR_CUDA, "cuTensorMapEncodeTiled(fp32 C^T) failed with CUresult %d", int(r));
            g.tma_store = 3;
        }
    } else if (c_panel_kg) {
        EncodeTiledFn enc = encode_tiled_fn();
        const long long all_rows = (long long)((N + 127) / 128) * c_panel_kg;
        if (all_rows > (1ll << 31) - 1) return fail(SD_ERR_TOO_LARGE, "panel matrix too large");
        cuuint64_t dims[2] = {128u, cuuint64_t(all_rows)};
        cuuint64_t strides[1] = {256u};
        cuuint32_t box[2] = {64u, 32u};
        cuuint32_t estr[2] = {1u, 1u};
        CUresult r = enc(&tc, dtype == SD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, C,
                         dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(SD_ERR_CUDA, "cuTensorMapEncodeTiled(C panels) failed with CUresult %d", int(r));
        g.tma_store = 1;
    } else if (c_cs == 1 && (c_rs & 7) == 0 && c_rs >= N && (reinterpret_cast<uintptr_t>(C) & 15) == 0) {
        EncodeTiledFn enc = encode_tiled_fn();
        cuuint64_t dims[2] = {cuuint64_t(N), cuuint64_t(M)};
        cuuint64_t strides[1] = {cuuint64_t(M > 1 ? c_rs * 2 : ((int64_t(N) * 2 + 15) & ~int64_t(15)))};
        cuuint32_t box[2] = {64u, 32u};
        cuuint32_t estr[2] = {1u, 1u};
        CUresult r = enc(&tc, dtype == SD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, C,
                         dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(SD_ERR_CUDA, "cuTensorMapEncodeTiled(C) failed with CUresult %d", int(r));
        g.tma_store = 1;
    } else if (c_rs == 1 && (c_cs & 7) == 0 && c_cs >= M && (reinterpret_cast<uintptr_t>(C) & 15) == 0) {
        EncodeTiledFn enc = encode_tiled_fn();
        cuuint64_t dims[2] = {cuuint64_t(M), cuuint64_t(N)};            // the transpose, row-major [N][M]
        cuuint64_t strides[1] = {cuuint64_t(N > 1 ? c_cs * 2 : ((int64_t(M) * 2 + 15) & ~int64_t(15)))};
        cuuint32_t box[2] = {32u, 64u};
        cuuint32_t estr[2] = {1u, 1u};
        CUresult r = enc(&tc, dtype == SD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, C,
                         dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(SD_ERR_CUDA, "cuTensorMapEncodeTiled(C^T) failed with CUresult %d", int(r));
        g.tma_store = 2;
    }
    // Epilogue warps (see MAX_EPI_WARPS): four when whole tiles have a long reduction to hide the epilogue behind,
    // eight otherwise.
    static const int epi_warps_env = [] {
        const char* e = getenv("SD_EPI_WARPS");            // tuning knob: 4 or 8 forces the choice
        const int v = e ? atoi(e) : 0;
        return (v == 4 || v == 8) ? v : 0;
    }();
    if (gather) {
        // four gather warps join the CTA, so the epilogue keeps four (the register budget of 352 threads)
        if (gather == 1 && !b_mn) return launch_variant<true, false, 1>(ta, tb, tc, g, grid, 4, st);
        if (gather == 1) return launch_variant<true, true, 1>(ta, tb, tc, g, grid, 4, st);
        if (b_mn) return launch_variant<false, true, 2>(ta, tb, tc, g, grid, 4, st);
        return launch_variant<false, false, 2>(ta, tb, tc, g, grid, 4, st);
    }
    const int epi_warps = epi_warps_env ? epi_warps_env : ((!g.split && k_tiles >= 24) ? 4 : MAX_EPI_WARPS);
    if (!a_mn && !b_mn) return launch_variant<false, false>(ta, tb, tc, g, grid, epi_warps, st);
    if (!a_mn && b_mn) return launch_variant<false, true>(ta, tb, tc, g, grid, epi_warps, st);
    if (a_mn && !b_mn) return launch_variant<true, false>(ta, tb, tc, g, grid, epi_warps, st);
    return launch_variant<true, true>(ta, tb, tc, g, grid, epi_warps, st);
}

// ------------------------------------------------------------------ built-in scratch
// Scratch of sd_gemm_dsd_static_scratch(): the same layout as a caller's workspace (counters, then one fp32
// partial tile per CTA) for at most kStaticScratchSlots CTAs: 8 KiB + 64 x 128 KiB = 8 200 KiB of device
// memory that every GPU which loads this library holds until the process exits.
constexpr int kStaticScratchSlots = 64;
static __device__ __align__(256) unsigned char sd_static_scratch[WS_FLAG_BYTES + kStaticScratchSlots * WS_SLOT_BYTES];

// Device address of the array on the current device.  In host code the array's name is only a stand-in for
// the symbol, not a device pointer: the address has to be asked for, once per device, with that device current.
static int static_scratch_address(void** out) {
    static std::mutex mu;
    static void* cached[64] = {};
    int dev = 0;
    SD_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 64 && cached[dev]) {
        *out = cached[dev];
        return SD_OK;
    }
    void* p = nullptr;
    SD_CUDA_TRY(cudaGetSymbolAddress(&p, sd_static_scratch));
    if (!p) return fail(SD_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the built-in scratch");
    if (dev < 64) cached[dev] = p;
    *out = p;
    return SD_OK;
}

}  // namespace sd

extern "C" {

int sd_gemm(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, void* C,
            int64_t c_rs, int64_t c_cs, int M, int N, int K, float scale, int dtype, void* workspace, int* status,
            void* stream) {
    return sd::run_gemm(sd::MODE_DENSE, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, nullptr, 0, scale, dtype,
                        workspace, status, stream);
}

int sd_gemm_dsd(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, void* C,
                int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, int plan_side, float scale,
                int dtype, void* workspace, int* status, void* stream) {
    return sd::run_gemm(sd::MODE_DSD, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, plan, plan_side, scale,
                        dtype, workspace, status, stream);
}

int sd_gemm_sdd(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, void* C,
                int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, float scale, int dtype,
                void* workspace, int* status, void* stream) {
    return sd::run_gemm(sd::MODE_SDD, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, plan, 0, scale, dtype,
                        workspace, status, stream);
}

int sd_gemm_sdd_kept(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, void* C,
                     int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, float scale, int dtype,
                     void* workspace, int* status, void* stream) {
    return sd::run_gemm(sd::MODE_SDD, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, plan, 0, scale, dtype,
                        workspace, status, stream, 0, /*zero_dropped=*/false);
}

int sd_gemm_sdd_kept_t(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, void* C,
                       int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, float scale, int dtype,
                       void* workspace, int* status, void* stream) {
    return sd::run_gemm(sd::MODE_SDD, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, plan, 0, scale, dtype,
                        workspace, status, stream, 0, /*zero_dropped=*/false, /*sdd_t=*/true);
}

int sd_gemm_dsd_panels(const void* P, int pixels, int kg, const void* B, int64_t b_rs, int64_t b_cs, void* C,
                       int64_t c_rs, int64_t c_cs, int N, const void* plan, int plan_side, float scale, int dtype,
                       void* workspace, int* status, void* stream) {
    if (plan_side != SD_PLAN_ROWS && plan_side != SD_PLAN_COLS)
        return sd::fail(SD_ERR_INVALID_ARG, "plan_side must be SD_PLAN_ROWS or SD_PLAN_COLS");
    const int M = plan_side == SD_PLAN_ROWS ? pixels : kg, K = plan_side == SD_PLAN_ROWS ? kg : pixels;
    return sd::run_gemm(sd::MODE_DSD, P, 0, 0, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, plan, plan_side, scale, dtype,
                        workspace, status, stream, 0, true, false, /*panels=*/1);
}

int sd_gemm_sdd_kept_t_panels(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs,
                              void* P, int kg, int pixels, int K, const void* plan, float scale, int dtype,
                              void* workspace, int* status, void* stream) {
    return sd::run_gemm(sd::MODE_SDD, A, a_rs, a_cs, B, b_rs, b_cs, P, 128, 1, kg, pixels, K, plan, 0, scale, dtype,
                        workspace, status, stream, 0, /*zero_dropped=*/false, /*sdd_t=*/true, /*panels=*/2);
}

// ---- fused convolution: the im2col matrix is gathered inside the GEMM kernel and never written to memory
static int make_conv_gather(sd::ConvGather* cv, const void* x, int N, int C, int H, int W, int R, int S, int pad_h,
                            int pad_w, int stride_h, int stride_w, int dil_h, int dil_w) {
    if (!x) return sd::fail(SD_ERR_INVALID_ARG, "x is null");
    if (!sd_conv_fused_supported(N, C, H, W, R, S, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w))
        return sd::fail(SD_ERR_INVALID_ARG,
                        "the fused convolution serves filters 3 wide with unit horizontal stride and dilation and one "
                        "column of padding on rows of 8, 16, 32 or 64 pixels; use the sd_im2col_kept path otherwise");
    if (reinterpret_cast<uintptr_t>(x) & 15) return sd::fail(SD_ERR_LAYOUT, "x must be 16-byte aligned");
    const int P = (H + 2 * pad_h - dil_h * (R - 1) - 1) / stride_h + 1;
    cv->x = static_cast<const unsigned short*>(x);
    cv->C = C; cv->H = H; cv->W = W; cv->R = R; cv->P = P;
    cv->stride_h = stride_h; cv->dil_h = dil_h; cv->pad_h = pad_h;
    cv->PQ = P * W; cv->HW = H * W;
    cv->k_real = C * R * 3;
    cv->pixels = N * P * W;
    cv->log2_w = W == 8 ? 3 : W == 16 ? 4 : W == 32 ? 5 : 6;
    sd::fast_div_constants(uint32_t(P * W), &cv->mul_pq, &cv->shr_pq);
    sd::fast_div_constants(uint32_t(R), &cv->mul_r, &cv->shr_r);
    cv->pass_dc[0] = cv->pass_dr[0] = 0;
    cv->pass_dc[1] = 4 / R; cv->pass_dr[1] = 4 % R;
    cv->pass_dc[2] = 8 / R; cv->pass_dr[2] = 8 % R;
    return SD_OK;
}

int sd_conv_fused_supported(int N, int C, int H, int W, int R, int S, int pad_h, int pad_w, int stride_h, int stride_w,
                            int dil_h, int dil_w) {
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || R <= 0 || S != 3) return 0;
    if (stride_w != 1 || dil_w != 1 || pad_w != 1 || stride_h <= 0 || dil_h <= 0 || pad_h < 0) return 0;
    if (W != 8 && W != 16 && W != 32 && W != 64) return 0;
    const long long P = ((long long)H + 2 * pad_h - (long long)dil_h * (R - 1) - 1) / stride_h + 1;
    if (P <= 0) return 0;
    if ((long long)N * P * W > (1ll << 30) || (long long)C * R * 3 > (1ll << 30)) return 0;
    if ((long long)N * C * H * W > (1ll << 31) - 1) return 0;
    return 1;
}

int sd_conv_dsd_fwd(const void* x, int N, int C, int H, int W, int R, int S, int pad_h, int pad_w, int stride_h,
                    int stride_w, int dil_h, int dil_w, const void* W2d, int64_t w_rs, int64_t w_cs, void* Y2d,
                    int64_t y_rs, int64_t y_cs, int Ko, const void* plan, float scale, int dtype, void* workspace,
                    int* status, void* stream) {
    sd::ConvGather cv;
    int rc = make_conv_gather(&cv, x, N, C, H, W, R, S, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w);
    if (rc) return rc;
    return sd::run_gemm(sd::MODE_DSD, nullptr, 0, 0, W2d, w_rs, w_cs, Y2d, y_rs, y_cs, cv.pixels, Ko, cv.k_real, plan,
                        SD_PLAN_ROWS, scale, dtype, workspace, status, stream, 0, true, false, 0, &cv, 1);
}

int sd_conv_dsd_dw(const void* x, int N, int C, int H, int W, int R, int S, int pad_h, int pad_w, int stride_h,
                   int stride_w, int dil_h, int dil_w, const void* dY2d, int64_t dy_rs, int64_t dy_cs, void* dW2d,
                   int64_t dw_rs, int64_t dw_cs, int Ko, const void* plan, float scale, int dtype, void* workspace,
                   int* status, void* stream) {
    sd::ConvGather cv;
    int rc = make_conv_gather(&cv, x, N, C, H, W, R, S, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w);
    if (rc) return rc;
    // dW2d^T [k, Ko] = (keep o col)^T [k, pixels] . dY2d^T [Ko, pixels]^T: B = dY2d^T, C = dW2d^T (strides swapped)
    return sd::run_gemm(sd::MODE_DSD, nullptr, 0, 0, dY2d, dy_cs, dy_rs, dW2d, dw_cs, dw_rs, cv.k_real, Ko, cv.pixels,
                        plan, SD_PLAN_COLS, scale, dtype, workspace, status, stream, 0, true, false, 0, &cv, 2);
}

int sd_gemm_dsd_relu(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, void* C,
                     int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, int plan_side, float scale,
                     int dtype, void* workspace, int* status, void* stream) {
    sd::GemmExtras ex;
    ex.act = 1;
    return sd::run_gemm(sd::MODE_DSD, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, plan, plan_side, scale,
                        dtype, workspace, status, stream, 0, true, false, 0, nullptr, 0, &ex);
}

int sd_gemm_dsd_f32(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, float* C,
                    int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, int plan_side, float scale,
                    int dtype, int accumulate, void* workspace, int* status, void* stream) {
    sd::GemmExtras ex;
    ex.out_f32 = 1;
    ex.out_acc = accumulate ? 1 : 0;
    return sd::run_gemm(sd::MODE_DSD, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, plan, plan_side, scale,
                        dtype, workspace, status, stream, 0, true, false, 0, nullptr, 0, &ex);
}

int sd_gemm_sdd_relu_mask(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, void* C,
                          int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, const void* X, int64_t x_rs,
                          float scale, int dtype, void* workspace, int* status, void* stream) {
    if (!X) return sd::fail(SD_ERR_INVALID_ARG, "X is null");
    sd::GemmExtras ex;
    ex.mask_src = X;
    ex.mask_rs = x_rs;
    return sd::run_gemm(sd::MODE_SDD, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, plan, 0, scale, dtype,
                        workspace, status, stream, 0, true, false, 0, nullptr, 0, &ex);
}

int sd_set_sm_margin(int sms) {
    if (sms < 0) return sd::fail(SD_ERR_INVALID_ARG, "the SM margin must not be negative (got %d)", sms);
    return sd::g_sm_margin.exchange(sms, std::memory_order_relaxed);
}

size_t sd_workspace_bytes(void) {
    int sms = 0;
    if (sd::sm_count_current_device(&sms) != SD_OK) return 0;
    if (sms > sd::WS_MAX_CTAS) sms = sd::WS_MAX_CTAS;
    return sd::WS_FLAG_BYTES + size_t(sms) * sd::WS_SLOT_BYTES;
}

int sd_workspace_init(void* workspace, void* stream) {
    if (!workspace) return sd::fail(SD_ERR_INVALID_ARG, "workspace is null");
    SD_CUDA_TRY(cudaMemsetAsync(workspace, 0, sd::WS_FLAG_BYTES, static_cast<cudaStream_t>(stream)));
    return SD_OK;
}

int sd_gemm_dsd_static_scratch(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs,
                               void* C, int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, int plan_side,
                               float scale, int dtype, int* status, void* stream) {
    void* scratch = nullptr;
    int rc = sd::static_scratch_address(&scratch);
    if (rc) return rc;
    // The array keeps whatever the previous call left.  Partial tiles are always written before they are
    // read, but the flags must start at zero, also after a launch that gave up on a wait.
    SD_CUDA_TRY(cudaMemsetAsync(scratch, 0, sd::WS_FLAG_BYTES, static_cast<cudaStream_t>(stream)));
    return sd::run_gemm(sd::MODE_DSD, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, plan, plan_side, scale,
                        dtype, scratch, status, stream, sd::kStaticScratchSlots);
}


int sd_check_status(const int* status, void* stream) {
    if (!status) return sd::fail(SD_ERR_INVALID_ARG, "status is null");
    int host = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SD_CUDA_TRY(cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, st));
    SD_CUDA_TRY(cudaStreamSynchronize(st));
    if (host != 0) return sd::fail(SD_ERR_TIMEOUT, "a device-side bounded wait expired (code %d)", host);
    return SD_OK;
}

}  // extern "C"
