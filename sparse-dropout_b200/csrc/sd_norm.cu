// LayerNorm forward and backward for the rows that feed the SparseDrop layers of the transformer consumers.
//
// The reference's models normalise with torch.nn.LayerNorm (eval/llm/model.py:72-74,113; eval/vit/model.py:11,53,
// 106-108) in fp32 under autocast and cast the result to 16 bits in front of every DropoutMM.  At the GPT config
// (16384 rows of 384) the stock backward spends 140 us per layer on the weight gradient alone; the two kernels here
// are plain HBM-bound passes: forward reads x once and writes y in the dtype its consumer wants (fp32 or 16 bits, so
// the cast disappears), backward reads x and dy once, writes dx, and leaves per-CTA partial sums of the weight and bias
// gradients that a second, tiny kernel adds up.
//
// Layout: one warp per row, each lane owns the float4 columns lane, lane + 32, ... (n a multiple of 4, at most
// 32 * 4 * kNormMaxVec = 1024), the row is held in registers between the statistics and the output pass.  The kernels
// are instantiated for 1, 2, 3, 4, 6 and 8 vectors per lane (VPL), so a narrow row does not pay the registers of a wide
// one and several CTAs fit an SM.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <atomic>

#include "sd_common.h"

namespace sd {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 4 values of a row in a 16-bit dtype <-> float4
template <int DT>
__device__ __forceinline__ float4 load4(const void* base, long long vec_index) {
    if (DT == SD_F32) return __ldg(reinterpret_cast<const float4*>(base) + vec_index);
    const uint2 q = __ldg(reinterpret_cast<const uint2*>(base) + vec_index);
    if (DT == SD_BF16)
        return make_float4(__uint_as_float(q.x << 16), __uint_as_float(q.x & 0xffff0000u), __uint_as_float(q.y << 16),
                           __uint_as_float(q.y & 0xffff0000u));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
template <int DT>
__device__ __forceinline__ void store4(void* base, long long vec_index, float4 v) {
    if (DT == SD_F32) {
        reinterpret_cast<float4*>(base)[vec_index] = v;
        return;
    }
    uint2 q;
    if (DT == SD_BF16) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        q.x = *reinterpret_cast<uint32_t*>(&a);
        q.y = *reinterpret_cast<uint32_t*>(&b);
    } else {
        __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        q.x = *reinterpret_cast<uint32_t*>(&a);
        q.y = *reinterpret_cast<uint32_t*>(&b);
    }
    reinterpret_cast<uint2*>(base)[vec_index] = q;
}

template <int OUT, int VPL>
__global__ void __launch_bounds__(kNormThreads)
layernorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                     void* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int n,
                     float eps) {
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, n_warps = (gridDim.x * blockDim.x) >> 5;
    const int nv = n >> 2;
    const float inv_n = 1.0f / float(n);
    for (int row = warp; row < rows; row += n_warps) {
        const float4* xr = reinterpret_cast<const float4*>(x) + (long long)row * nv;
        float4 v[VPL];
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int c = lane + 32 * j;
            v[j] = c < nv ? __ldg(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        }
        const float mean = warp_sum(s) * inv_n;
        float q = 0.f;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            if (lane + 32 * j < nv) {
                const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                q += (a * a + b * b) + (c * c + d * d);
            }
        }
        const float rstd = rsqrtf(warp_sum(q) * inv_n + eps);
        if (lane == 0) {
            mean_out[row] = mean;
            rstd_out[row] = rstd;
        }
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int c = lane + 32 * j;
            if (c < nv) {
                const float4 g = __ldg(reinterpret_cast<const float4*>(gamma) + c);
                float4 o = make_float4((v[j].x - mean) * rstd * g.x, (v[j].y - mean) * rstd * g.y,
                                       (v[j].z - mean) * rstd * g.z, (v[j].w - mean) * rstd * g.w);
                if (beta) {
                    const float4 b = __ldg(reinterpret_cast<const float4*>(beta) + c);
                    o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
                }
                store4<OUT>(y, (long long)row * nv + c, o);
            }
        }
    }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)), g = dy * gamma, xhat = (x - mean) * rstd; per-CTA partial sums of
// dgamma = sum_rows dy * xhat and dbeta = sum_rows dy go to partials[blockIdx.x][2][n].
template <int DYT, int VPL>
__global__ void __launch_bounds__(kNormThreads)
layernorm_bwd_kernel(const float* __restrict__ x, const void* __restrict__ dy, const float* __restrict__ gamma,
                     const float* __restrict__ mean_in, const float* __restrict__ rstd_in, float* __restrict__ dx,
                     float* __restrict__ partials, int rows, int n) {
    __shared__ float acc[2 * 32 * 4 * VPL];
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, n_warps = (gridDim.x * blockDim.x) >> 5;
    const int nv = n >> 2;
    const float inv_n = 1.0f / float(n);
    for (int i = threadIdx.x; i < 2 * n; i += blockDim.x) acc[i] = 0.f;
    __syncthreads();
    float4 dg[VPL], db[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) dg[j] = db[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int row = warp; row < rows; row += n_warps) {
        const float mean = __ldg(mean_in + row), rstd = __ldg(rstd_in + row);
        float4 xh[VPL], g[VPL];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int c = lane + 32 * j;
            if (c < nv) {
                const float4 xv = __ldg(reinterpret_cast<const float4*>(x) + (long long)row * nv + c);
                const float4 d = load4<DYT>(dy, (long long)row * nv + c);
                const float4 gm = __ldg(reinterpret_cast<const float4*>(gamma) + c);
                xh[j] = make_float4((xv.x - mean) * rstd, (xv.y - mean) * rstd, (xv.z - mean) * rstd, (xv.w - mean) * rstd);
                g[j] = make_float4(d.x * gm.x, d.y * gm.y, d.z * gm.z, d.w * gm.w);
                s1 += (g[j].x + g[j].y) + (g[j].z + g[j].w);
                s2 += (g[j].x * xh[j].x + g[j].y * xh[j].y) + (g[j].z * xh[j].z + g[j].w * xh[j].w);
                dg[j].x += d.x * xh[j].x; dg[j].y += d.y * xh[j].y; dg[j].z += d.z * xh[j].z; dg[j].w += d.w * xh[j].w;
                db[j].x += d.x; db[j].y += d.y; db[j].z += d.z; db[j].w += d.w;
            } else {
                xh[j] = g[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        const float c1 = warp_sum(s1) * inv_n, c2 = warp_sum(s2) * inv_n;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int c = lane + 32 * j;
            if (c < nv)
                reinterpret_cast<float4*>(dx)[(long long)row * nv + c] =
                    make_float4(rstd * (g[j].x - c1 - xh[j].x * c2), rstd * (g[j].y - c1 - xh[j].y * c2),
                                rstd * (g[j].z - c1 - xh[j].z * c2), rstd * (g[j].w - c1 - xh[j].w * c2));
        }
    }
    // the CTA's eight warps add their column sums in shared memory, then the CTA writes one partial row
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int c = (lane + 32 * j) * 4;
        if (c < n) {
            atomicAdd(acc + c, dg[j].x); atomicAdd(acc + c + 1, dg[j].y); atomicAdd(acc + c + 2, dg[j].z); atomicAdd(acc + c + 3, dg[j].w);
            atomicAdd(acc + n + c, db[j].x); atomicAdd(acc + n + c + 1, db[j].y); atomicAdd(acc + n + c + 2, db[j].z);
            atomicAdd(acc + n + c + 3, db[j].w);
        }
    }
    __syncthreads();
    float* out = partials + (long long)blockIdx.x * 2 * n;
    for (int i = threadIdx.x; i < 2 * n; i += blockDim.x) out[i] = acc[i];
}

// Column sums of partials[parts][2n]: thread (tx, ty) adds rows ty, ty + 32, ... of column blockIdx.x * 32 + tx, four
// rows at a time so that their loads are in flight together.
__global__ void __launch_bounds__(1024)
layernorm_bwd_reduce_kernel(const float* __restrict__ partials, int parts, int n, float* __restrict__ dgamma,
                            float* __restrict__ dbeta, int accumulate) {
    __shared__ float red[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + tx;
    const long long stride = 2ll * n;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (col < 2 * n) {
        int p = ty;
        for (; p + 96 < parts; p += 128) {
            s0 += __ldg(partials + p * stride + col);
            s1 += __ldg(partials + (p + 32) * stride + col);
            s2 += __ldg(partials + (p + 64) * stride + col);
            s3 += __ldg(partials + (p + 96) * stride + col);
        }
        for (; p < parts; p += 32) s0 += __ldg(partials + p * stride + col);
    }
    red[ty][tx] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    if (ty == 0 && col < 2 * n) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 32; ++k) t += red[k][tx];
        float* dst = col < n ? dgamma + col : (dbeta ? dbeta + (col - n) : nullptr);
        if (dst) *dst = accumulate ? *dst + t : t;
    }
}

static int norm_grid(int rows, int* grid) {
    int sms = 0;
    const int rc = sm_count_current_device(&sms);
    if (rc) return rc;
    const long long blocks = ((long long)rows + 7) / 8;
    *grid = int(blocks < (long long)sms * 4 ? blocks : (long long)sms * 4);
    return SD_OK;
}

// smallest instantiated VPL that covers n / 4 float4 per row
static int norm_vpl(int n) {
    const int need = ((n >> 2) + 31) >> 5;
    const int have[6] = {1, 2, 3, 4, 6, 8};
    for (int v : have)
        if (need <= v) return v;
    return 0;
}

#define SD_NORM_DISPATCH_VPL(vpl, CALL)                                    \
    switch (vpl) {                                                         \
        case 1: { constexpr int V = 1; CALL; } break;                      \
        case 2: { constexpr int V = 2; CALL; } break;                      \
        case 3: { constexpr int V = 3; CALL; } break;                      \
        case 4: { constexpr int V = 4; CALL; } break;                      \
        case 6: { constexpr int V = 6; CALL; } break;                      \
        default: { constexpr int V = 8; CALL; } break;                     \
    }

// Backward launch: at most as many CTAs as are resident at once (a second, partly filled wave would run at a fraction
// of the memory-level parallelism), never more than the workspace was sized for (`grid`, see norm_grid).
template <int DYT, int V>
static int launch_norm_bwd(int grid, cudaStream_t st, const float* x, const void* dy, const float* gamma, const float* mean,
                           const float* rstd, float* dx, float* partials, int rows, int n, int* grid_used) {
    static std::atomic<int> per_sm_cached{0};   // the same on every device this process sees (one GPU type per node)
    int sms = 0;
    const int rc = sm_count_current_device(&sms);
    if (rc) return rc;
    int per_sm = per_sm_cached.load(std::memory_order_relaxed);
    if (per_sm == 0) {
        int nb = 0;
        SD_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, layernorm_bwd_kernel<DYT, V>, kNormThreads, 0));
        per_sm = nb > 0 ? nb : 1;
        per_sm_cached.store(per_sm, std::memory_order_relaxed);
    }
    if (grid > sms * per_sm) grid = sms * per_sm;
    layernorm_bwd_kernel<DYT, V><<<grid, kNormThreads, 0, st>>>(x, dy, gamma, mean, rstd, dx, partials, rows, n);
    *grid_used = grid;
    return SD_OK;
}

static int check_norm_args(const void* x, int rows, int n) {
    if (!x) return fail(SD_ERR_INVALID_ARG, "x is null");
    if (rows <= 0 || n <= 0) return fail(SD_ERR_INVALID_ARG, "rows and n must be positive (got %d, %d)", rows, n);
    if ((n & 3) || n > 128 * kNormMaxVec)
        return fail(SD_ERR_LAYOUT, "the normalised width must be a multiple of 4 and at most %d (got %d)", 128 * kNormMaxVec, n);
    if (reinterpret_cast<uintptr_t>(x) & 15) return fail(SD_ERR_LAYOUT, "x must be 16-byte aligned");
    return SD_OK;
}

}  // namespace sd

extern "C" {

int sd_layernorm_fwd(const float* x, int rows, int n, const float* gamma, const float* beta, float eps, void* y,
                     int y_dtype, float* mean, float* rstd, void* stream) {
    int rc = sd::check_norm_args(x, rows, n);
    if (rc) return rc;
    if (!gamma || !y || !mean || !rstd) return sd::fail(SD_ERR_INVALID_ARG, "gamma, y, mean and rstd must not be null");
    if ((reinterpret_cast<uintptr_t>(y) & (y_dtype == SD_F32 ? 15 : 7)) || (reinterpret_cast<uintptr_t>(gamma) & 15) ||
        (beta && (reinterpret_cast<uintptr_t>(beta) & 15)))
        return sd::fail(SD_ERR_LAYOUT, "y, gamma and beta must be aligned to four elements");
    int grid = 0;
    rc = sd::norm_grid(rows, &grid);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int vpl = sd::norm_vpl(n);
    if (y_dtype == SD_F32) {
        SD_NORM_DISPATCH_VPL(vpl, (sd::layernorm_fwd_kernel<SD_F32, V><<<grid, sd::kNormThreads, 0, st>>>(x, gamma, beta, y, mean, rstd, rows, n, eps)))
    } else if (y_dtype == SD_BF16) {
        SD_NORM_DISPATCH_VPL(vpl, (sd::layernorm_fwd_kernel<SD_BF16, V><<<grid, sd::kNormThreads, 0, st>>>(x, gamma, beta, y, mean, rstd, rows, n, eps)))
    } else if (y_dtype == SD_F16) {
        SD_NORM_DISPATCH_VPL(vpl, (sd::layernorm_fwd_kernel<SD_F16, V><<<grid, sd::kNormThreads, 0, st>>>(x, gamma, beta, y, mean, rstd, rows, n, eps)))
    } else {
        return sd::fail(SD_ERR_INVALID_ARG, "y_dtype must be SD_F16, SD_BF16 or SD_F32");
    }
    SD_CUDA_TRY(cudaGetLastError());
    return SD_OK;
}

size_t sd_layernorm_bwd_workspace_bytes(int rows, int n) {
    int grid = 0;
    if (rows <= 0 || n <= 0 || sd::norm_grid(rows, &grid) != SD_OK) return 0;
    return size_t(grid) * 2 * size_t(n) * sizeof(float);
}

int sd_layernorm_bwd(const float* x, const void* dy, int dy_dtype, const float* gamma, const float* mean,
                     const float* rstd, int rows, int n, float* dx, float* dgamma, float* dbeta, int accumulate,
                     void* workspace, void* stream) {
    int rc = sd::check_norm_args(x, rows, n);
    if (rc) return rc;
    if (!dy || !gamma || !mean || !rstd || !dx || !dgamma || !workspace)
        return sd::fail(SD_ERR_INVALID_ARG, "dy, gamma, mean, rstd, dx, dgamma and workspace must not be null");
    if ((reinterpret_cast<uintptr_t>(dy) & (dy_dtype == SD_F32 ? 15 : 7)) || (reinterpret_cast<uintptr_t>(dx) & 15) ||
        (reinterpret_cast<uintptr_t>(gamma) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 15))
        return sd::fail(SD_ERR_LAYOUT, "dy, dx, gamma and workspace must be aligned to four elements");
    int grid = 0;
    rc = sd::norm_grid(rows, &grid);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* partials = static_cast<float*>(workspace);
    int parts = grid;
    const int vpl = sd::norm_vpl(n);
    if (dy_dtype == SD_F32) {
        SD_NORM_DISPATCH_VPL(vpl, (rc = sd::launch_norm_bwd<SD_F32, V>(grid, st, x, dy, gamma, mean, rstd, dx, partials, rows, n, &parts)))
    } else if (dy_dtype == SD_BF16) {
        SD_NORM_DISPATCH_VPL(vpl, (rc = sd::launch_norm_bwd<SD_BF16, V>(grid, st, x, dy, gamma, mean, rstd, dx, partials, rows, n, &parts)))
    } else if (dy_dtype == SD_F16) {
        SD_NORM_DISPATCH_VPL(vpl, (rc = sd::launch_norm_bwd<SD_F16, V>(grid, st, x, dy, gamma, mean, rstd, dx, partials, rows, n, &parts)))
    } else {
        return sd::fail(SD_ERR_INVALID_ARG, "dy_dtype must be SD_F16, SD_BF16 or SD_F32");
    }
    if (rc) return rc;
    SD_CUDA_TRY(cudaGetLastError());
    sd::layernorm_bwd_reduce_kernel<<<(2 * n + 31) / 32, 1024, 0, st>>>(partials, parts, n, dgamma, dbeta, accumulate);
    SD_CUDA_TRY(cudaGetLastError());
    return SD_OK;
}

}  // extern "C"
