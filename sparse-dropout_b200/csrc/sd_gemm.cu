// Persistent, warp-specialised tcgen05 GEMM for sm_100a that walks only kept tiles.
//
// One kernel template serves the three products of a SparseDrop linear layer and the dense
// comparator; D[MM, NN] = scale * A[MM, KK] . B[NN, KK]^T throughout:
//   dense : every 128-wide K tile                      (flash_dropout/cuda/src/gemm.cuh:100-140)
//   DSD   : per 128-row block of A, only the K tiles on that block's kept list
//           (flash_dropout/cuda/src/matmul_dsd.cuh:18-68 re-reads a bool mask every k-step and
//           `continue`s; here the producer warp never even visits a dropped tile)
//   SDD   : only kept 128x128 output tiles are computed, two per work item; dropped tiles are
//           zero-filled by the otherwise idle epilogue warps
//           (flash_dropout/cuda/src/matmul_sdd.cuh:18-67 launches a CTA per tile, kept or not)
//
// CTA = 6 warps on one SM, 128 x 256 output tile, 64-wide K stages in a 4-deep TMA ring:
//   warp 0    producer : one lane issues cp.async.bulk.tensor loads (no multicast) into
//                        128B-swizzled shared memory, completion on `full` mbarriers
//   warp 1    MMA      : one lane issues tcgen05.mma (M128 N256 K16, fp32 accumulate in TMEM),
//                        tcgen05.commit releases ring stages and publishes accumulators
//   warps 2-5 epilogue : tcgen05.ld the accumulator (two 256-column TMEM buffers, so the
//                        epilogue of tile i overlaps the main loop of tile i+1), scale, convert,
//                        store to global memory
// Both operands may be K-major (reduction dimension contiguous) or MN-major; that is the
// (row|col)-major x (row|col)-major operand matrix of flash_dropout/cuda/src/gemm_binding.cu:51-53.
//
// Every wait is bounded (sd_ptx.cuh: mbar_wait); on expiry the CTA records a code in the status
// word, every role leaves its loop, TMEM is freed and the kernel returns normally.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

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
constexpr int GEMM_SMEM = TILE_SMEM + 1024 /*align*/ + 256 /*barriers*/;
constexpr int GEMM_THREADS = 192;
constexpr int TMEM_COLS = 512;

enum GemmMode { MODE_DENSE = 0, MODE_DSD = 1, MODE_SDD = 2 };
enum StatusCode { ST_PRODUCER = 1, ST_MMA_FULL = 2, ST_MMA_ACC = 3, ST_EPILOGUE = 4 };

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
    const int* order;                // DSD: row blocks, heaviest first (may be null)
    const int* items;                // SDD: (row block, col tile 0, col tile 1 or -1)
    const int* n_items;
    const int* zero_pairs;           // SDD: dropped (row block, col tile) pairs
    const int* n_zero;
    int* status;
    uint32_t idesc256, idesc128;
};

struct Work {
    int a_row, b_row0, b_row1;   // element coordinates along the operands' MN dimension; b_row1 < 0: absent
    int nk;                      // number of 128-wide K tiles
    const int* klist;            // their indices, or null for 0..nk-1
};

__device__ __forceinline__ int num_work(const GemmArgs& g) {
    return g.mode == MODE_SDD ? __ldg(g.n_items) : g.n_row_blocks * g.n_col_tiles;
}

__device__ __forceinline__ Work get_work(const GemmArgs& g, int t) {
    Work w;
    if (g.mode == MODE_SDD) {
        const int mb = __ldg(g.items + 3 * t), c0 = __ldg(g.items + 3 * t + 1), c1 = __ldg(g.items + 3 * t + 2);
        w.a_row = mb * 128;
        w.b_row0 = c0 * 128;
        w.b_row1 = c1 >= 0 ? c1 * 128 : -1;
        w.nk = (g.KK + 127) >> 7;
        w.klist = nullptr;
    } else {
        const int rbi = t / g.n_col_tiles, nt = t - rbi * g.n_col_tiles;
        const int rb = g.order ? __ldg(g.order + rbi) : rbi;
        w.a_row = rb * 128;
        w.b_row0 = nt * BN;
        w.b_row1 = (nt * BN + 128 < g.NN) ? nt * BN + 128 : -1;
        if (g.mode == MODE_DSD) {
            const int beg = __ldg(g.list_ptr + rb);
            w.nk = __ldg(g.list_ptr + rb + 1) - beg;
            w.klist = g.list_idx + beg;
        } else {
            w.nk = (g.KK + 127) >> 7;
            w.klist = nullptr;
        }
    }
    return w;
}

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

// Thread holds 32 consecutive fp32 values of output row `row`, columns [col, col+32).
__device__ __forceinline__ void store_chunk(const GemmArgs& g, bool vec_ok, int row, int col, const uint32_t (&r)[32]) {
    if (row >= g.MM || col >= g.NN) return;
    unsigned short* C = static_cast<unsigned short*>(g.C);
    if (vec_ok && col + 32 <= g.NN) {
        uint4* dst = reinterpret_cast<uint4*>(C + (long long)row * g.c_rs + col);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack2(__uint_as_float(r[8 * v + 0]) * g.scale, __uint_as_float(r[8 * v + 1]) * g.scale, g.is_bf16);
            o.y = pack2(__uint_as_float(r[8 * v + 2]) * g.scale, __uint_as_float(r[8 * v + 3]) * g.scale, g.is_bf16);
            o.z = pack2(__uint_as_float(r[8 * v + 4]) * g.scale, __uint_as_float(r[8 * v + 5]) * g.scale, g.is_bf16);
            o.w = pack2(__uint_as_float(r[8 * v + 6]) * g.scale, __uint_as_float(r[8 * v + 7]) * g.scale, g.is_bf16);
            dst[v] = o;
        }
    } else {
        // ragged edge, unaligned rows, or a column-major result (consecutive lanes = consecutive
        // rows, so a column-major store is a 64-byte contiguous segment per warp instruction)
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col + j < g.NN)
                C[(long long)row * g.c_rs + (long long)(col + j) * g.c_cs] = cvt1(__uint_as_float(r[j]) * g.scale, g.is_bf16);
    }
}

// Zero a 128 x 128 output tile with the 128 epilogue threads (tid in [0,128)).
__device__ __forceinline__ void zero_tile(const GemmArgs& g, bool vec_ok, int tid, int row0, int col0) {
    unsigned short* C = static_cast<unsigned short*>(g.C);
    if (vec_ok && row0 + 128 <= g.MM && col0 + 128 <= g.NN) {
        const int cchunk = tid & 15, rsub = tid >> 4;
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
            const int row = row0 + i * 8 + rsub;
            *reinterpret_cast<uint4*>(C + (long long)row * g.c_rs + col0 + cchunk * 8) = make_uint4(0, 0, 0, 0);
        }
    } else if (g.c_rs == 1) {
        for (int j = 0; j < 128; ++j)
            if (row0 + tid < g.MM && col0 + j < g.NN) C[(long long)(col0 + j) * g.c_cs + row0 + tid] = 0;
    } else {
        for (int i = 0; i < 128; ++i)
            if (row0 + i < g.MM && col0 + tid < g.NN) C[(long long)(row0 + i) * g.c_rs + (long long)(col0 + tid) * g.c_cs] = 0;
    }
}

// ------------------------------------------------------------------ the kernel
template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
sparsedrop_gemm_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                       const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t tiles = (raw_addr + 1023u) & ~1023u;   // 128B swizzle atoms need 1024-byte alignment
    uint8_t* aligned = smem_raw + (tiles - raw_addr);
    uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + TILE_SMEM);
    // bars[0..3] full, [4..7] empty, [8..9] tmem_full, [10..11] tmem_empty
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 13);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, 4);
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmapA);
        tma_prefetch_desc(&tmapB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_work = num_work(g);

    if (warp == 0) {
        // ============================== producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < n_work; t += gridDim.x) {
                const Work w = get_work(g, t);
                const uint32_t tx = A_BYTES + (w.b_row1 >= 0 ? B_BYTES : B_HALF_BYTES);
                for (int i = 0; ok && i < w.nk; ++i) {
                    const int kb = w.klist ? __ldg(w.klist + i) : i;
                    for (int h = 0; h < 2; ++h) {
                        const int k = kb * 128 + h * BK;
                        if (k >= g.KK) break;
                        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, g.status, ST_PRODUCER)) { ok = false; break; }
                        const uint32_t full = bar_full + 8 * stage;
                        mbar_arrive_expect_tx(full, tx);
                        const uint32_t sA = tiles + stage * STAGE_BYTES, sB = sA + A_BYTES;
                        if (!A_MN) {
                            tma_load_2d(sA, &tmapA, full, k, w.a_row);
                        } else {
                            tma_load_2d(sA, &tmapA, full, w.a_row, k);
                            tma_load_2d(sA + MN_ATOM_BYTES, &tmapA, full, w.a_row + 64, k);
                        }
                        if (!B_MN) {
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
        if (lane == 0) {
            constexpr uint64_t A_HI = A_MN ? make_smem_desc_hi(MN_ATOM_BYTES, 1024) : make_smem_desc_hi(16, 1024);
            constexpr uint64_t B_HI = B_MN ? make_smem_desc_hi(MN_ATOM_BYTES, 1024) : make_smem_desc_hi(16, 1024);
            constexpr uint32_t A_KSTEP = A_MN ? 2048 : 32;   // bytes per 16-wide K step
            constexpr uint32_t B_KSTEP = B_MN ? 2048 : 32;
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < n_work; t += gridDim.x) {
                const Work w = get_work(g, t);
                if (w.nk == 0) continue;
                if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, g.status, ST_MMA_ACC)) break;
                tc_fence_after();
                const uint32_t d = tmem_base + acc * BN;
                const uint32_t idesc = w.b_row1 >= 0 ? g.idesc256 : g.idesc128;
                uint32_t accumulate = 0;
                for (int i = 0; ok && i < w.nk; ++i) {
                    const int kb = w.klist ? __ldg(w.klist + i) : i;
                    for (int h = 0; h < 2; ++h) {
                        if (kb * 128 + h * BK >= g.KK) break;
                        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status, ST_MMA_FULL)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t sA = tiles + stage * STAGE_BYTES, sB = sA + A_BYTES;
#pragma unroll
                        for (int j = 0; j < BK / 16; ++j) {
                            umma_f16(d, make_smem_desc(sA + j * A_KSTEP, A_HI), make_smem_desc(sB + j * B_KSTEP, B_HI),
                                     idesc, accumulate);
                            accumulate = 1;
                        }
                        umma_commit(bar_empty + 8 * stage);
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    }
                }
                if (!ok) break;
                umma_commit(bar_tfull + 8 * acc);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
        __syncwarp();
    } else {
        // ============================== epilogue (warps 2..5 own TMEM lane quadrants 2,3,0,1)
        const int quad = warp & 3;
        const int etid = quad * 32 + lane;   // 0..127, also the row inside the tile this thread owns
        const bool vec_ok = g.c_cs == 1 && (g.c_rs & 7) == 0 && (reinterpret_cast<uintptr_t>(g.C) & 15) == 0;
        if (g.mode == MODE_SDD) {
            const int nz = __ldg(g.n_zero);
            for (int z = blockIdx.x; z < nz; z += gridDim.x)
                zero_tile(g, vec_ok, etid, __ldg(g.zero_pairs + 2 * z) * 128, __ldg(g.zero_pairs + 2 * z + 1) * 128);
        }
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = blockIdx.x; t < n_work; t += gridDim.x) {
            const Work w = get_work(g, t);
            if (w.nk == 0) {
                zero_tile(g, vec_ok, etid, w.a_row, w.b_row0);
                if (w.b_row1 >= 0) zero_tile(g, vec_ok, etid, w.a_row, w.b_row1);
                continue;
            }
            if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, g.status, ST_EPILOGUE)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + acc * BN + (uint32_t(quad * 32) << 16);
            const int row = w.a_row + etid;
            const int nchunks = w.b_row1 >= 0 ? 8 : 4;
            for (int c = 0; c < nchunks; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_ld_wait();
                const int col = c < 4 ? w.b_row0 + c * 32 : w.b_row1 + (c - 4) * 32;
                store_chunk(g, vec_ok, row, col, r);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
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
    *mn_major = !k_major;
    return SD_OK;
}

template <bool A_MN, bool B_MN>
static int launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int grid, cudaStream_t st) {
    static bool configured[64] = {};
    int dev = 0;
    SD_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        SD_CUDA_TRY(cudaFuncSetAttribute(sparsedrop_gemm_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GEMM_SMEM));
        configured[dev] = true;
    } else if (dev >= 64) {
        SD_CUDA_TRY(cudaFuncSetAttribute(sparsedrop_gemm_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GEMM_SMEM));
    }
    sparsedrop_gemm_kernel<A_MN, B_MN><<<grid, GEMM_THREADS, GEMM_SMEM, st>>>(ta, tb, g);
    SD_CUDA_TRY(cudaGetLastError());
    return SD_OK;
}

struct PlanView {
    const int *header, *row_ptr, *col_idx, *col_ptr, *row_idx, *row_order, *col_order, *sdd_items, *drop_pairs;
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
    return v;
}

static int run_gemm(int mode, const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs,
                    void* C, int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, int plan_side,
                    float scale, int dtype, int* status, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return fail(SD_ERR_INVALID_ARG, "M, N, K must be positive (got %d, %d, %d)", M, N, K);
    if (dtype != SD_F16 && dtype != SD_BF16) return fail(SD_ERR_INVALID_ARG, "dtype must be SD_F16 or SD_BF16");
    if (!C) return fail(SD_ERR_INVALID_ARG, "C is null");
    if (c_rs != 1 && c_cs != 1) return fail(SD_ERR_LAYOUT, "C must be row or column major");
    if (mode != MODE_DENSE && !plan) return fail(SD_ERR_INVALID_ARG, "plan is null");
    if (mode == MODE_DSD && plan_side != SD_PLAN_ROWS && plan_side != SD_PLAN_COLS)
        return fail(SD_ERR_INVALID_ARG, "plan_side must be SD_PLAN_ROWS or SD_PLAN_COLS");

    // Bind the device's primary context to this thread before the first driver-API call: a thread that
    // has made no runtime call yet (e.g. an autograd worker) has no current context and
    // cuTensorMapEncodeTiled would fail with CUDA_ERROR_INVALID_CONTEXT.
    int dev = 0;
    SD_CUDA_TRY(cudaGetDevice(&dev));
    SD_CUDA_TRY(cudaSetDevice(dev));

    CUtensorMap ta, tb;
    bool a_mn = false, b_mn = false;
    int rc = make_operand_map(&ta, &a_mn, "A", A, a_rs, a_cs, M, K, dtype);
    if (rc) return rc;
    rc = make_operand_map(&tb, &b_mn, "B", B, b_rs, b_cs, N, K, dtype);
    if (rc) return rc;

    GemmArgs g{};
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

    int sms = 0;
    rc = sm_count_current_device(&sms);
    if (rc) return rc;
    int grid = sms;
    if (mode == MODE_DSD) {
        const int kb = (K + 127) / 128;
        if (plan_side == SD_PLAN_ROWS) {
            PlanView v = view_plan(plan, g.n_row_blocks, kb);
            g.list_ptr = v.row_ptr; g.list_idx = v.col_idx; g.order = v.row_order;
        } else {
            PlanView v = view_plan(plan, kb, g.n_row_blocks);
            g.list_ptr = v.col_ptr; g.list_idx = v.row_idx; g.order = v.col_order;
        }
    } else if (mode == MODE_SDD) {
        PlanView v = view_plan(plan, g.n_row_blocks, (N + 127) / 128);
        g.items = v.sdd_items; g.n_items = v.header + H_SDD_ITEMS;
        g.zero_pairs = v.drop_pairs; g.n_zero = v.header + H_NDROP;
    }
    if (mode != MODE_SDD) {
        const long long tiles = (long long)g.n_row_blocks * g.n_col_tiles;
        if (tiles < grid) grid = int(tiles);
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!a_mn && !b_mn) return launch_variant<false, false>(ta, tb, g, grid, st);
    if (!a_mn && b_mn) return launch_variant<false, true>(ta, tb, g, grid, st);
    if (a_mn && !b_mn) return launch_variant<true, false>(ta, tb, g, grid, st);
    return launch_variant<true, true>(ta, tb, g, grid, st);
}

}  // namespace sd

extern "C" {

int sd_gemm(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, void* C,
            int64_t c_rs, int64_t c_cs, int M, int N, int K, float scale, int dtype, int* status, void* stream) {
    return sd::run_gemm(sd::MODE_DENSE, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, nullptr, 0, scale, dtype,
                        status, stream);
}

int sd_gemm_dsd(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, void* C,
                int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, int plan_side, float scale,
                int dtype, int* status, void* stream) {
    return sd::run_gemm(sd::MODE_DSD, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, plan, plan_side, scale,
                        dtype, status, stream);
}

int sd_gemm_sdd(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, void* C,
                int64_t c_rs, int64_t c_cs, int M, int N, int K, const void* plan, float scale, int dtype,
                int* status, void* stream) {
    return sd::run_gemm(sd::MODE_SDD, A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, N, K, plan, 0, scale, dtype,
                        status, stream);
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
