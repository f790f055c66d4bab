// im2col / col2im stages of the SparseDrop convolution, restricted to the kept 128x128 blocks.
//
// The im2col matrix of flash_dropout/functional/im2col_conv2d.py:17-20 has M = N*P*Q rows and K = C*R*S
// columns, k = c*R*S + r*S + s.  It is stored K-outer here ("colT": row k holds all M entries of column k,
// leading dimension ldm), because consecutive m are consecutive pixels of the NCHW input, so both the gather
// and the store run along the contiguous direction and the GEMM kernel takes colT.T as an MN-major operand.
// Only blocks the plan keeps are ever written or read: at p = 0.5 half of the 2 x 302 MB an unfold
// (flash_dropout/functional/im2col_conv2d.py:17) moves.  Both kernels are pure data movement: HBM-bound.
//
// The reference's own CUDA im2col (flash_dropout/cuda/src/im2col.cuh:17-72) is an NHWC scatter that was never
// built; nothing is taken from it.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sd_common.h"
#include "sd_plan.cuh"

namespace sd {

struct ConvGeom {
    int N, C, H, W, R, S, P, Q;
    int pad_h, pad_w, stride_h, stride_w, dil_h, dil_w;
    int M, K;           // N*P*Q, C*R*S
    long long ldm;      // columns of colT that exist (>= M, multiple of 8)
    int Rb, Cb;         // plan grid: ceil(M/128) x ceil(K/128) (K as the GEMM sees it)
    long long kstride;  // elements from one k-row to the next: ldm, or 128 in the panel layout
    long long pstride;  // panel layout ([M/128][k_gemm][128], a kept block is one 32 KB run): elements per panel; else 0
};

// Offset of element (k, m) of the K-outer im2col matrix.  Eight consecutive m starting at a multiple of 8 are
// contiguous in either layout.
__device__ __forceinline__ long long col_off(const ConvGeom& g, long long k, long long m) {
    return g.pstride ? (m >> 7) * g.pstride + k * 128 + (m & 127) : k * g.ldm + m;
}

constexpr int kConvThreads = 256;

// Elements [e0, e0 + 8) of a row of `len` 16-bit elements, zero outside [0, len).  The row starts 16-byte aligned
// and len is a multiple of 8, so each of the (at most two) aligned 8-element chunks the window touches lies either
// entirely inside the row or entirely outside it: two 16-byte loads and a funnel shift replace eight 2-byte loads.
__device__ __forceinline__ void load8_shifted(const unsigned short* __restrict__ row, int e0, int len, uint32_t (&out)[4]) {
    const int a = e0 & ~7, sh = e0 - a;
    uint4 c0 = make_uint4(0, 0, 0, 0), c1 = make_uint4(0, 0, 0, 0);
    if (a >= 0 && a < len) c0 = __ldg(reinterpret_cast<const uint4*>(row + a));
    if (sh && a + 8 >= 0 && a + 8 < len) c1 = __ldg(reinterpret_cast<const uint4*>(row + a + 8));
    uint32_t w0 = c0.x, w1 = c0.y, w2 = c0.z, w3 = c0.w, w4 = c1.x, w5 = c1.y, w6 = c1.z, w7 = c1.w;
    const int ws = sh >> 1;
    if (ws & 1) { w0 = w1; w1 = w2; w2 = w3; w3 = w4; w4 = w5; w5 = w6; w6 = w7; }
    if (ws & 2) { w0 = w2; w1 = w3; w2 = w4; w3 = w5; w4 = w6; }
    const uint32_t sb = (sh & 1) * 16;
    out[0] = __funnelshift_r(w0, w1, sb);
    out[1] = __funnelshift_r(w1, w2, sb);
    out[2] = __funnelshift_r(w2, w3, sb);
    out[3] = __funnelshift_r(w3, w4, sb);
}

// Fast im2col for unit horizontal stride with W % 8 == 0 and Q % 8 == 0: the 8 output pixels a thread owns sit in
// one output row, so each k-row is one shifted 8-element window of one input row.
__global__ void __launch_bounds__(kConvThreads) im2col_kept_rows_kernel(const unsigned short* __restrict__ x,
                                                                        unsigned short* __restrict__ colT, ConvGeom g,
                                                                        const int* __restrict__ kept_pairs,
                                                                        const int* __restrict__ n_kept) {
    const int total = kept_pairs ? __ldg(n_kept) : g.Rb * g.Cb;
    const int mgrp = threadIdx.x & 15, ksub = threadIdx.x >> 4;
    const int PQ = g.P * g.Q, HW = g.H * g.W, RS = g.R * g.S;
    for (int t = blockIdx.x; t < total; t += gridDim.x) {
        const int mb = kept_pairs ? __ldg(kept_pairs + 2 * t) : t / g.Cb;
        const int kb = kept_pairs ? __ldg(kept_pairs + 2 * t + 1) : t - (t / g.Cb) * g.Cb;
        const int m0 = mb * 128 + mgrp * 8;
        if (m0 >= g.ldm) continue;
        const bool live = m0 < g.M;                      // M % 8 == 0 here, so the group is all in or all out
        const int n = live ? m0 / PQ : 0, pq = m0 - n * PQ, p = pq / g.Q, q0 = pq - p * g.Q;
        const unsigned short* xn = x + (long long)n * g.C * HW;
        const int hbase = p * g.stride_h - g.pad_h, wbase = q0 - g.pad_w;
        // (c, r*S + s) of this thread's first k-row; every pass advances k by 16 without dividing by C*R*S again
        int c = (kb * 128 + ksub) / RS, rs = (kb * 128 + ksub) - c * RS;
        const int c16 = 16 / RS, rs16 = 16 - c16 * RS;
#pragma unroll 2
        for (int pass = 0; pass < 8; ++pass) {
            const int k = kb * 128 + pass * 16 + ksub;
            if (k >= g.K) break;
            const int r = rs / g.S, s = rs - r * g.S;
            const int h = hbase + r * g.dil_h;
            uint32_t o[4] = {0, 0, 0, 0};
            if (live && (unsigned)h < (unsigned)g.H)
                load8_shifted(xn + (long long)c * HW + (long long)h * g.W, wbase + s * g.dil_w, g.W, o);
            *reinterpret_cast<uint4*>(colT + col_off(g, k, m0)) = make_uint4(o[0], o[1], o[2], o[3]);
            c += c16;
            rs += rs16;
            if (rs >= RS) { rs -= RS; ++c; }
        }
    }
}

// Fastest im2col: filters 3 wide with unit horizontal stride and dilation and one column of padding (so Q == W),
// rows of 8..128 pixels that divide 128.  The three taps s = 0, 1, 2 of one (c, r) read the same input row shifted
// by -1, 0, +1: a thread loads the aligned 8-pixel chunk once, borrows the one pixel on either side from its
// neighbour lanes (which own the neighbouring chunks of the same image row) and writes three k-rows.
__global__ void __launch_bounds__(kConvThreads) im2col_kept_s3_kernel(const unsigned short* __restrict__ x,
                                                                      unsigned short* __restrict__ colT, ConvGeom g,
                                                                      const int* __restrict__ kept_pairs,
                                                                      const int* __restrict__ n_kept) {
    const int total = kept_pairs ? __ldg(n_kept) : g.Rb * g.Cb;
    const int mgrp = threadIdx.x & 15, tsub = threadIdx.x >> 4;
    const int PQ = g.P * g.Q, HW = g.H * g.W;
    for (int t = blockIdx.x; t < total; t += gridDim.x) {
        const int mb = kept_pairs ? __ldg(kept_pairs + 2 * t) : t / g.Cb;
        const int kb = kept_pairs ? __ldg(kept_pairs + 2 * t + 1) : t - (t / g.Cb) * g.Cb;
        const int m0 = mb * 128 + mgrp * 8;
        const bool in_ld = m0 < g.ldm;                   // all lanes stay in the loop: they trade pixels below
        const bool live = m0 < g.M;                      // M % 8 == 0 here, so the group is all in or all out
        const int n = live ? m0 / PQ : 0, pq = m0 - n * PQ, p = pq / g.Q, q0 = pq - p * g.Q;
        const unsigned short* xn = x + (long long)n * g.C * HW;
        const int hbase = p * g.stride_h - g.pad_h;
        const bool has_left = q0 > 0, has_right = q0 + 8 < g.Q;
        const int k_lo = kb * 128, k_hi = min(k_lo + 128, g.K);
        // (c, r) pairs whose three k-rows 3 * (c * R + r) + s touch [k_lo, k_hi); the same number of passes for
        // every thread, because the shuffles below need whole warps
        const int cr_end = (k_hi + 2) / 3;
        for (int cr0 = k_lo / 3; cr0 < cr_end; cr0 += 16) {
            const int cr = cr0 + tsub;
            const bool valid = cr < cr_end;
            const int c = cr / g.R, r = cr - c * g.R;
            const int h = hbase + r * g.dil_h;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (valid && live && (unsigned)h < (unsigned)g.H)
                v = __ldg(reinterpret_cast<const uint4*>(xn + (long long)c * HW + (long long)h * g.W + q0));
            uint32_t left = __shfl_up_sync(0xffffffffu, v.w, 1), right = __shfl_down_sync(0xffffffffu, v.x, 1);
            if (!has_left) left = 0;
            if (!has_right) right = 0;
            if (!valid || !in_ld) continue;
            const uint32_t a0 = __funnelshift_r(v.x, v.y, 16), a1 = __funnelshift_r(v.y, v.z, 16),
                           a2 = __funnelshift_r(v.z, v.w, 16);
            unsigned short* dst = colT + col_off(g, 3 * cr, m0);
            if (3 * cr >= k_lo)
                *reinterpret_cast<uint4*>(dst) = make_uint4(__funnelshift_r(left, v.x, 16), a0, a1, a2);
            if (3 * cr + 1 >= k_lo && 3 * cr + 1 < k_hi) *reinterpret_cast<uint4*>(dst + g.kstride) = v;
            if (3 * cr + 2 < k_hi)
                *reinterpret_cast<uint4*>(dst + 2 * g.kstride) = make_uint4(a0, a1, a2, __funnelshift_r(v.w, right, 16));
        }
    }
}

// One CTA per kept block (grid-stride): 128 k-rows x 128 m-columns of colT.  Thread t owns the 8 consecutive m
// starting at (t % 16) * 8 and visits k-rows (t / 16) + 16 * pass.
__global__ void __launch_bounds__(kConvThreads) im2col_kept_kernel(const unsigned short* __restrict__ x,
                                                                   unsigned short* __restrict__ colT, ConvGeom g,
                                                                   const int* __restrict__ kept_pairs,
                                                                   const int* __restrict__ n_kept) {
    const int total = kept_pairs ? __ldg(n_kept) : g.Rb * g.Cb;
    const int mgrp = threadIdx.x & 15, ksub = threadIdx.x >> 4;
    const int PQ = g.P * g.Q, HW = g.H * g.W, RS = g.R * g.S;
    for (int t = blockIdx.x; t < total; t += gridDim.x) {
        const int mb = kept_pairs ? __ldg(kept_pairs + 2 * t) : t / g.Cb;
        const int kb = kept_pairs ? __ldg(kept_pairs + 2 * t + 1) : t - (t / g.Cb) * g.Cb;
        const int m0 = mb * 128 + mgrp * 8;
        if (m0 >= g.ldm) continue;
        // decode the 8 output pixels once
        long long base[8];
        int hb[8], wb[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int m = m0 + j;
            if (m < g.M) {
                const int n = m / PQ, pq = m - n * PQ, p = pq / g.Q, q = pq - p * g.Q;
                base[j] = (long long)n * g.C * HW;
                hb[j] = p * g.stride_h - g.pad_h;
                wb[j] = q * g.stride_w - g.pad_w;
            } else {
                base[j] = 0;
                hb[j] = -(1 << 28);   // never in range: the padding columns of colT are zero
                wb[j] = 0;
            }
        }
#pragma unroll 2
        for (int pass = 0; pass < 8; ++pass) {
            const int k = kb * 128 + pass * 16 + ksub;
            if (k >= g.K) break;
            const int c = k / RS, rs = k - c * RS, r = rs / g.S, s = rs - r * g.S;
            const int hoff = r * g.dil_h, woff = s * g.dil_w;
            const unsigned short* xc = x + (long long)c * HW;
            unsigned short v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int h = hb[j] + hoff, w = wb[j] + woff;
                const bool in = (unsigned)h < (unsigned)g.H && (unsigned)w < (unsigned)g.W;
                v[j] = in ? __ldg(xc + base[j] + (long long)h * g.W + w) : (unsigned short)0;
            }
            uint4 o;
            o.x = v[0] | (uint32_t(v[1]) << 16);
            o.y = v[2] | (uint32_t(v[3]) << 16);
            o.z = v[4] | (uint32_t(v[5]) << 16);
            o.w = v[6] | (uint32_t(v[7]) << 16);
            *reinterpret_cast<uint4*>(colT + col_off(g, k, m0)) = o;
        }
    }
}

__device__ __forceinline__ float to_float(unsigned short v, int is_bf16) {
    return is_bf16 ? __bfloat162float(__ushort_as_bfloat16(v)) : __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ unsigned short from_float(float f, int is_bf16) {
    return is_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(f)) : __half_as_ushort(__float2half_rn(f));
}

// Adjoint of the kept-block im2col: dx[n,c,h,w] = sum over the filter taps (r,s) that map (h,w) to an output
// pixel (p,q) of dcolT[k(c,r,s)][m(n,p,q)], skipping dropped blocks (their entries are zero by definition).
// One thread per input element, consecutive threads along w, so every tap is a coalesced read along m.
__global__ void __launch_bounds__(kConvThreads) col2im_kept_kernel(const unsigned short* __restrict__ dcolT,
                                                                   unsigned short* __restrict__ dx, ConvGeom g,
                                                                   const unsigned char* __restrict__ tile_mask,
                                                                   int is_bf16) {
    const long long total = (long long)g.N * g.C * g.H * g.W;
    const int PQ = g.P * g.Q, RS = g.R * g.S;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int w = int(i % g.W);
        long long rest = i / g.W;
        const int h = int(rest % g.H);
        rest /= g.H;
        const int c = int(rest % g.C), n = int(rest / g.C);
        float acc = 0.f;
        for (int r = 0; r < g.R; ++r) {
            const int hh = h + g.pad_h - r * g.dil_h;
            if (hh < 0 || hh % g.stride_h) continue;
            const int p = hh / g.stride_h;
            if (p >= g.P) continue;
            for (int s = 0; s < g.S; ++s) {
                const int ww = w + g.pad_w - s * g.dil_w;
                if (ww < 0 || ww % g.stride_w) continue;
                const int q = ww / g.stride_w;
                if (q >= g.Q) continue;
                const int m = n * PQ + p * g.Q + q, k = c * RS + r * g.S + s;
                if (tile_mask && tile_mask[(m >> 7) * g.Cb + (k >> 7)]) continue;
                acc += to_float(__ldg(dcolT + col_off(g, k, m)), is_bf16);
            }
        }
        dx[i] = from_float(acc, is_bf16);
    }
}

// Fast col2im for unit strides with W % 8 == 0 and Q % 8 == 0: a thread owns 8 consecutive w of one (n, c, h);
// every filter tap is one shifted 8-element window of one dcolT row, whose aligned chunks each lie in one block.
template <bool IS_BF16>
__global__ void __launch_bounds__(kConvThreads) col2im_kept_rows_kernel(const unsigned short* __restrict__ dcolT,
                                                                        unsigned short* __restrict__ dx, ConvGeom g,
                                                                        const unsigned char* __restrict__ tile_mask) {
    const int WG = g.W >> 3;
    const unsigned total = unsigned(g.N) * g.C * g.H * WG;       // the host checks that this fits 32 bits
    const int PQ = g.P * g.Q, RS = g.R * g.S;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int wg = int(i % WG);
        unsigned rest = i / WG;
        const int h = int(rest % g.H);
        rest /= g.H;
        const int c = int(rest % g.C), n = int(rest / g.C);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < g.R; ++r) {
            const int p = h + g.pad_h - r * g.dil_h;
            if ((unsigned)p >= (unsigned)g.P) continue;
            for (int s = 0; s < g.S; ++s) {
                const int k = c * RS + r * g.S + s;
                const int q0 = wg * 8 + g.pad_w - s * g.dil_w;        // output column that w = wg*8 fed through tap s
                const int a = q0 & ~7, sh = q0 - a;
                const long long mrow = (long long)n * PQ + (long long)p * g.Q;
                const unsigned short* rowa = dcolT + col_off(g, k, mrow + a);           // used only when the chunk exists
                const unsigned short* rowb = dcolT + col_off(g, k, mrow + a + 8);
                // chunk validity: inside [0, Q) and in a kept block
                uint4 c0 = make_uint4(0, 0, 0, 0), c1 = make_uint4(0, 0, 0, 0);
                if (a >= 0 && a < g.Q && !(tile_mask && tile_mask[((mrow + a) >> 7) * g.Cb + (k >> 7)]))
                    c0 = __ldg(reinterpret_cast<const uint4*>(rowa));
                if (sh && a + 8 >= 0 && a + 8 < g.Q && !(tile_mask && tile_mask[((mrow + a + 8) >> 7) * g.Cb + (k >> 7)]))
                    c1 = __ldg(reinterpret_cast<const uint4*>(rowb));
                uint32_t w0 = c0.x, w1 = c0.y, w2 = c0.z, w3 = c0.w, w4 = c1.x, w5 = c1.y, w6 = c1.z, w7 = c1.w;
                const int ws = sh >> 1;
                if (ws & 1) { w0 = w1; w1 = w2; w2 = w3; w3 = w4; w4 = w5; w5 = w6; w6 = w7; }
                if (ws & 2) { w0 = w2; w1 = w3; w2 = w4; w3 = w5; w4 = w6; }
                const uint32_t sb = (sh & 1) * 16;
                const uint32_t o[4] = {__funnelshift_r(w0, w1, sb), __funnelshift_r(w1, w2, sb),
                                       __funnelshift_r(w2, w3, sb), __funnelshift_r(w3, w4, sb)};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (IS_BF16) {                               // bf16 -> fp32 is a 16-bit shift
                        acc[2 * j] += __uint_as_float(o[j] << 16);
                        acc[2 * j + 1] += __uint_as_float(o[j] & 0xffff0000u);
                    } else {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&o[j]));
                        acc[2 * j] += f.x;
                        acc[2 * j + 1] += f.y;
                    }
                }
            }
        }
        uint32_t out[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (IS_BF16) {
                __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                out[j] = *reinterpret_cast<uint32_t*>(&v);
            } else {
                __half2 v = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
                out[j] = *reinterpret_cast<uint32_t*>(&v);
            }
        }
        *reinterpret_cast<uint4*>(dx + (long long)i * 8) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// Fastest col2im: the adjoint of im2col_kept_s3_kernel under the same conditions plus unit vertical stride.  A thread
// owns 8 consecutive w of one (n, c, h) and reads, for each of the R x 3 taps, the aligned 8-pixel chunk of the tap's
// dcolT row; taps s = 0 and s = 2 are that chunk shifted by one pixel, the pixel that falls off going to the
// neighbour lane (which owns the neighbouring 8 pixels of the same image row).
template <bool IS_BF16>
__global__ void __launch_bounds__(kConvThreads) col2im_kept_s3_kernel(const unsigned short* __restrict__ dcolT,
                                                                      unsigned short* __restrict__ dx, ConvGeom g,
                                                                      const unsigned char* __restrict__ tile_mask) {
    const int WG = g.W >> 3;                                     // lanes per image row; divides 32
    const unsigned total = unsigned(g.N) * g.C * g.H * WG;       // the host checks that this fits 32 bits
    const unsigned total_up = (total + 31u) & ~31u;              // whole warps run the loop: they trade pixels
    const int PQ = g.P * g.Q;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total_up; i += gridDim.x * blockDim.x) {
        const bool live = i < total;
        const int wg = int(i % WG);
        unsigned rest = i / WG;
        const int h = int(rest % g.H);
        rest /= g.H;
        const int c = live ? int(rest % g.C) : 0, n = live ? int(rest / g.C) : 0;
        const bool has_left = wg > 0, has_right = wg + 1 < WG;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < g.R; ++r) {
            const int p = h + g.pad_h - r * g.dil_h;
            const bool row_ok = live && (unsigned)p < (unsigned)g.P;
            const long long m = (long long)n * PQ + (long long)p * g.Q + wg * 8;
            const int k0 = (c * g.R + r) * 3;
            float f[3][8];
#pragma unroll
            for (int s = 0; s < 3; ++s) {
                const int k = k0 + s;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (row_ok && !(tile_mask && tile_mask[(m >> 7) * g.Cb + (k >> 7)]))
                    v = __ldg(reinterpret_cast<const uint4*>(dcolT + col_off(g, k, m)));
                const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (IS_BF16) {                               // bf16 -> fp32 is a 16-bit shift
                        f[s][2 * j] = __uint_as_float(wv[j] << 16);
                        f[s][2 * j + 1] = __uint_as_float(wv[j] & 0xffff0000u);
                    } else {
                        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&wv[j]));
                        f[s][2 * j] = t.x;
                        f[s][2 * j + 1] = t.y;
                    }
                }
            }
            // dx[w] += dcol[s][q = w + 1 - s]: tap 0 reads one pixel to the right, tap 2 one to the left
            float from_right = __shfl_down_sync(0xffffffffu, f[0][0], 1);
            float from_left = __shfl_up_sync(0xffffffffu, f[2][7], 1);
            if (!has_right) from_right = 0.f;
            if (!has_left) from_left = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc[j] += f[1][j];
                acc[j] += j < 7 ? f[0][j + 1] : from_right;
                acc[j] += j > 0 ? f[2][j - 1] : from_left;
            }
        }
        if (!live) continue;
        uint32_t out[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (IS_BF16) {
                __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                out[j] = *reinterpret_cast<uint32_t*>(&v);
            } else {
                __half2 v = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
                out[j] = *reinterpret_cast<uint32_t*>(&v);
            }
        }
        *reinterpret_cast<uint4*>(dx + (long long)i * 8) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// The same for 3 x 3 filters, unrolled over all nine taps: first the nine block-mask bytes, then the nine chunk loads
// (independent of one another, so one memory round trip covers them all), then the arithmetic.
template <bool IS_BF16>
__global__ void __launch_bounds__(kConvThreads) col2im_kept_3x3_kernel(const unsigned short* __restrict__ dcolT,
                                                                       unsigned short* __restrict__ dx, ConvGeom g,
                                                                       const unsigned char* __restrict__ tile_mask) {
    const int WG = g.W >> 3, wg_bits = 31 - __clz(WG);           // lanes per image row: a power of two up to 16
    const unsigned total = unsigned(g.N) * g.C * g.H * WG;       // the host checks that this fits 32 bits
    const unsigned total_up = (total + 31u) & ~31u;              // whole warps run the loop: they trade pixels
    const int PQ = g.P * g.Q;
    const long long tap_step = g.kstride;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total_up; i += gridDim.x * blockDim.x) {
        const bool live = i < total;
        const int wg = int(i & (WG - 1));
        unsigned rest = i >> wg_bits;
        const int h = int(rest % g.H);
        rest /= g.H;
        const int c = live ? int(rest % g.C) : 0, n = live ? int(rest / g.C) : 0;
        const int p0 = h + g.pad_h, k0 = c * 9;
        const long long m0 = (long long)n * PQ + wg * 8;
        const unsigned short* src[3];                             // tap (r, 0) of each filter row
        bool ok[9];
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const int p = p0 - r * g.dil_h;
            const bool row_ok = live && (unsigned)p < (unsigned)g.P;
            const long long m = m0 + (long long)p * g.Q;
            src[r] = dcolT + col_off(g, k0 + 3 * r, m);
            const int mrow = int(m >> 7) * g.Cb;
#pragma unroll
            for (int s = 0; s < 3; ++s)
                ok[3 * r + s] = row_ok && !(tile_mask && __ldg(tile_mask + mrow + ((k0 + 3 * r + s) >> 7)));
        }
        uint4 v[9];
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int s = 0; s < 3; ++s)
                v[3 * r + s] = ok[3 * r + s] ? __ldg(reinterpret_cast<const uint4*>(src[r] + s * tap_step))
                                             : make_uint4(0, 0, 0, 0);
        const bool has_left = wg > 0, has_right = wg + 1 < WG;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            float f[3][8];
#pragma unroll
            for (int s = 0; s < 3; ++s) {
                const uint32_t wv[4] = {v[3 * r + s].x, v[3 * r + s].y, v[3 * r + s].z, v[3 * r + s].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (IS_BF16) {                               // bf16 -> fp32 is a 16-bit shift
                        f[s][2 * j] = __uint_as_float(wv[j] << 16);
                        f[s][2 * j + 1] = __uint_as_float(wv[j] & 0xffff0000u);
                    } else {
                        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&wv[j]));
                        f[s][2 * j] = t.x;
                        f[s][2 * j + 1] = t.y;
                    }
                }
            }
            // dx[w] += dcol[s][q = w + 1 - s]: tap 0 reads one pixel to the right, tap 2 one to the left
            float from_right = __shfl_down_sync(0xffffffffu, f[0][0], 1);
            float from_left = __shfl_up_sync(0xffffffffu, f[2][7], 1);
            if (!has_right) from_right = 0.f;
            if (!has_left) from_left = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc[j] += f[1][j];
                acc[j] += j < 7 ? f[0][j + 1] : from_right;
                acc[j] += j > 0 ? f[2][j - 1] : from_left;
            }
        }
        if (!live) continue;
        uint32_t out[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (IS_BF16) {
                __nv_bfloat162 t = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                out[j] = *reinterpret_cast<uint32_t*>(&t);
            } else {
                __half2 t = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
                out[j] = *reinterpret_cast<uint32_t*>(&t);
            }
        }
        *reinterpret_cast<uint4*>(dx + (long long)i * 8) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

static int make_geom(ConvGeom* g, int N, int C, int H, int W, int R, int S, int pad_h, int pad_w, int stride_h,
                     int stride_w, int dil_h, int dil_w, int64_t ldm, int k_gemm, bool panels = false) {
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || R <= 0 || S <= 0)
        return fail(SD_ERR_INVALID_ARG, "conv sizes must be positive");
    if (stride_h <= 0 || stride_w <= 0 || dil_h <= 0 || dil_w <= 0 || pad_h < 0 || pad_w < 0)
        return fail(SD_ERR_INVALID_ARG, "stride and dilation must be positive, padding non-negative");
    const int P = (H + 2 * pad_h - dil_h * (R - 1) - 1) / stride_h + 1;
    const int Q = (W + 2 * pad_w - dil_w * (S - 1) - 1) / stride_w + 1;
    if (P <= 0 || Q <= 0) return fail(SD_ERR_INVALID_ARG, "the filter does not fit the padded input");
    const long long M = (long long)N * P * Q, K = (long long)C * R * S;
    if (M > (1ll << 30) || K > (1ll << 30)) return fail(SD_ERR_TOO_LARGE, "im2col matrix too large (M=%lld, K=%lld)", M, K);
    if (panels) ldm = ((M + 127) / 128) * 128;      // whole panels exist
    if (ldm < M || (ldm & 7)) return fail(SD_ERR_LAYOUT, "ldm (%lld) must be >= N*P*Q (%lld) and a multiple of 8", (long long)ldm, M);
    if (k_gemm < K) return fail(SD_ERR_INVALID_ARG, "k_gemm (%d) must be >= C*R*S (%lld)", k_gemm, K);
    *g = ConvGeom{N, C, H, W, R, S, P, Q, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, int(M), int(K), ldm,
                  int((M + 127) / 128), (k_gemm + 127) / 128, panels ? 128 : ldm, panels ? (long long)k_gemm * 128 : 0};
    return SD_OK;
}

}  // namespace sd

static int im2col_kept_impl(const void* x, int N, int C, int H, int W, int R, int S, int pad_h, int pad_w, int stride_h,
                            int stride_w, int dil_h, int dil_w, void* colT, int64_t ldm, int k_gemm, const void* plan,
                            void* stream, bool panels) {
    if (!x || !colT) return sd::fail(SD_ERR_INVALID_ARG, "x or colT is null");
    if ((reinterpret_cast<uintptr_t>(colT) & 15)) return sd::fail(SD_ERR_LAYOUT, "colT must be 16-byte aligned");
    sd::ConvGeom g;
    int rc = sd::make_geom(&g, N, C, H, W, R, S, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, ldm, k_gemm, panels);
    if (rc) return rc;
    const int *pairs = nullptr, *n_kept = nullptr;
    if (plan) {
        const sd_plan_layout L = sd::plan_layout(g.Rb, g.Cb);
        const unsigned char* b = static_cast<const unsigned char*>(plan);
        pairs = reinterpret_cast<const int*>(b + L.kept_pairs);
        n_kept = reinterpret_cast<const int*>(b + L.header) + sd::H_NNZ;
    }
    int sms = 0;
    rc = sd::sm_count_current_device(&sms);
    if (rc) return rc;
    long long blocks = (long long)g.Rb * g.Cb;
    int grid = int(blocks < (long long)sms * 8 ? blocks : (long long)sms * 8);
    const bool rows_path = stride_w == 1 && (W & 7) == 0 && (g.Q & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    const bool s3_path = rows_path && S == 3 && dil_w == 1 && pad_w == 1 && W <= 128 && 128 % W == 0;
    if (s3_path)
        sd::im2col_kept_s3_kernel<<<grid, sd::kConvThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const unsigned short*>(x), static_cast<unsigned short*>(colT), g, pairs, n_kept);
    else if (rows_path)
        sd::im2col_kept_rows_kernel<<<grid, sd::kConvThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const unsigned short*>(x), static_cast<unsigned short*>(colT), g, pairs, n_kept);
    else
        sd::im2col_kept_kernel<<<grid, sd::kConvThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const unsigned short*>(x), static_cast<unsigned short*>(colT), g, pairs, n_kept);
    SD_CUDA_TRY(cudaGetLastError());
    return SD_OK;
}

static int col2im_kept_impl(const void* dcolT, int64_t ldm, int k_gemm, int N, int C, int H, int W, int R, int S, int pad_h,
                            int pad_w, int stride_h, int stride_w, int dil_h, int dil_w, void* dx, const void* plan,
                            int dtype, void* stream, bool panels) {
    if (!dcolT || !dx) return sd::fail(SD_ERR_INVALID_ARG, "dcolT or dx is null");
    if (dtype != SD_F16 && dtype != SD_BF16) return sd::fail(SD_ERR_INVALID_ARG, "dtype must be SD_F16 or SD_BF16");
    sd::ConvGeom g;
    int rc = sd::make_geom(&g, N, C, H, W, R, S, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, ldm, k_gemm, panels);
    if (rc) return rc;
    const unsigned char* mask = nullptr;
    if (plan) mask = static_cast<const unsigned char*>(plan) + sd::plan_layout(g.Rb, g.Cb).mask;
    int sms = 0;
    rc = sd::sm_count_current_device(&sms);
    if (rc) return rc;
    const bool rows_path = stride_w == 1 && stride_h == 1 && (W & 7) == 0 && (g.Q & 7) == 0 &&
                           ((reinterpret_cast<uintptr_t>(dcolT) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0 &&
                           (long long)N * C * H * (W / 8) < (1ll << 31);
    const long long total = (long long)N * C * H * (rows_path ? W / 8 : W);
    long long blocks = (total + sd::kConvThreads - 1) / sd::kConvThreads;
    int grid = int(blocks < (long long)sms * 16 ? blocks : (long long)sms * 16);
    const bool s3_path = rows_path && S == 3 && dil_w == 1 && pad_w == 1 && W <= 128 && 128 % W == 0;
    if (s3_path && R == 3 && dtype == SD_BF16)
        sd::col2im_kept_3x3_kernel<true><<<grid, sd::kConvThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const unsigned short*>(dcolT), static_cast<unsigned short*>(dx), g, mask);
    else if (s3_path && R == 3)
        sd::col2im_kept_3x3_kernel<false><<<grid, sd::kConvThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const unsigned short*>(dcolT), static_cast<unsigned short*>(dx), g, mask);
    else if (s3_path && dtype == SD_BF16)
        sd::col2im_kept_s3_kernel<true><<<grid, sd::kConvThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const unsigned short*>(dcolT), static_cast<unsigned short*>(dx), g, mask);
    else if (s3_path)
        sd::col2im_kept_s3_kernel<false><<<grid, sd::kConvThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const unsigned short*>(dcolT), static_cast<unsigned short*>(dx), g, mask);
    else if (rows_path && dtype == SD_BF16)
        sd::col2im_kept_rows_kernel<true><<<grid, sd::kConvThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const unsigned short*>(dcolT), static_cast<unsigned short*>(dx), g, mask);
    else if (rows_path)
        sd::col2im_kept_rows_kernel<false><<<grid, sd::kConvThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const unsigned short*>(dcolT), static_cast<unsigned short*>(dx), g, mask);
    else
        sd::col2im_kept_kernel<<<grid, sd::kConvThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const unsigned short*>(dcolT), static_cast<unsigned short*>(dx), g, mask, dtype == SD_BF16);
    SD_CUDA_TRY(cudaGetLastError());
    return SD_OK;
}

extern "C" {

int sd_im2col_kept(const void* x, int N, int C, int H, int W, int R, int S, int pad_h, int pad_w, int stride_h,
                   int stride_w, int dil_h, int dil_w, void* colT, int64_t ldm, int k_gemm, const void* plan,
                   void* stream) {
    return im2col_kept_impl(x, N, C, H, W, R, S, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, colT, ldm, k_gemm, plan,
                            stream, false);
}

int sd_im2col_kept_panels(const void* x, int N, int C, int H, int W, int R, int S, int pad_h, int pad_w, int stride_h,
                          int stride_w, int dil_h, int dil_w, void* col_panels, int k_gemm, const void* plan,
                          void* stream) {
    return im2col_kept_impl(x, N, C, H, W, R, S, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, col_panels, 0, k_gemm,
                            plan, stream, true);
}

int sd_col2im_kept(const void* dcolT, int64_t ldm, int k_gemm, int N, int C, int H, int W, int R, int S, int pad_h,
                   int pad_w, int stride_h, int stride_w, int dil_h, int dil_w, void* dx, const void* plan, int dtype,
                   void* stream) {
    return col2im_kept_impl(dcolT, ldm, k_gemm, N, C, H, W, R, S, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, dx,
                            plan, dtype, stream, false);
}

int sd_col2im_kept_panels(const void* dcol_panels, int k_gemm, int N, int C, int H, int W, int R, int S, int pad_h,
                          int pad_w, int stride_h, int stride_w, int dil_h, int dil_w, void* dx, const void* plan,
                          int dtype, void* stream) {
    return col2im_kept_impl(dcol_panels, 0, k_gemm, N, C, H, W, R, S, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
                            dx, plan, dtype, stream, true);
}

}  // extern "C"
