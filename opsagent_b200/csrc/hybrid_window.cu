// hybrid_window.cu — windowed softmax attention over cached keys and values for the hybrid decoder family (API: hybrid_kernels.hpp), and the RMS
// norm pair that feeds a layer whose mixer and feed-forward read separate norms of the same residual.
//
// One mechanism with its constants as parameters (HyWinAttn): `heads` query heads on `kv_heads` key/value heads; `maps` score maps per head
// (2 = differential attention: the head's query and key rows hold [map 1 | map 2], both maps weigh the same values, and the head's output is
// (a1 - lambda a2) scaled to unit RMS times out_scale); a sliding window of `window` positions plus the first `keep_first` positions of the
// sequence; an optional RMS norm of every query / key map; an optional sink logit per head that only enlarges the softmax denominator; a
// sigmoid output gate per channel or per head.  Softmax, norms and gates are fp32 in both element types.
#include "hybrid_common.cuh"
#include "hybrid_kernels.hpp"

namespace oa {

namespace {

using namespace hyk;

// out1[t] = x[row] / sqrt(mean(x[row]^2) + eps) * w1 (and out2 with w2): one read of the residual row for both norms
template <typename TA>
__global__ void __launch_bounds__(256) hy_rmsnorm_pair_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const float* __restrict__ w1, TA* __restrict__ out1,
                                                              const float* __restrict__ w2, TA* __restrict__ out2, int ldo, int W, float eps) {
    HY_PDL();
    __shared__ float red[32];
    const int t = blockIdx.x; const float* xr = x + (long long)(rows ? rows[t] : t) * W;
    float s = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float v = xr[c]; s = fmaf(v, v, s); }
    const float rr = 1.0f / sqrtf(block_sum(s, red) / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = xr[c] * rr;
        stf(out1 + (long long)t * ldo + c, v * w1[c]);
        if (out2) stf(out2 + (long long)t * ldo + c, v * w2[c]);
    }
}

// Per row: RMS norm of every query map in place (qk_norm), keys (normed alike) and values into the row's cache slot [kv_heads maps dim | kv_heads vdim].
// One warp per vector.
template <typename TA>
__global__ void __launch_bounds__(128) hy_win_prep_kernel(HyWinAttn a, TA* __restrict__ q, int ldq, const TA* __restrict__ k, const TA* __restrict__ v, int ldkv,
                                                          const float* __restrict__ qw, const float* __restrict__ kw, float eps, TA* __restrict__ cache, HyRows r) {
    HY_PDL();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, D = a.dim;
    const int nq = a.qk_norm ? a.heads * a.maps : 0, nk = k ? a.kv_heads * a.maps : 0, KW = a.kv_heads * a.maps * D, CW = KW + a.kv_heads * a.vdim;
    TA* crow = cache + (long long)r.slots[t] * CW;
    for (int u = warp; u < nq + nk; u += 4) {
        const bool is_q = u < nq; const int i = is_q ? u : u - nq;
        const TA* src = is_q ? q + (long long)t * ldq + (long long)i * D : k + (long long)t * ldkv + (long long)i * D;
        TA* dst = is_q ? q + (long long)t * ldq + (long long)i * D : crow + (long long)i * D;
        float rr = 1.f;
        if (a.qk_norm) {
            float ss = 0.f;
            for (int c = lane; c < D; c += 32) { const float x = ldf(src + c); ss = fmaf(x, x, ss); }
            rr = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
        }
        const float* w = is_q ? qw : kw;
        for (int c = lane; c < D; c += 32) stf(dst + c, a.qk_norm ? ldf(src + c) * rr * w[c] : ldf(src + c));
    }
    if (v) for (int c = threadIdx.x; c < a.kv_heads * a.vdim; c += blockDim.x) crow[KW + c] = v[(long long)t * ldkv + c];
}

// The visible keys of a query at position p, in the order every kernel walks them: the kept first positions that the window no longer
// covers, then the window.  n = count; key(i) = i-th visible position.
struct WinKeys {
    int n_keep, lo, n;
    __device__ __forceinline__ WinKeys(int p, int window, int keep_first) { lo = max(0, p - window + 1); n_keep = min(keep_first, lo); n = n_keep + (p - lo + 1); }
    __device__ __forceinline__ int key(int i) const { return i < n_keep ? i : lo + (i - n_keep); }
};

constexpr int WIN_MAXV = 8;       // value channels per lane: vdim <= 32 * WIN_MAXV
// Plain form, any sizes, both element types: one CTA per (row, head); its four warps take the visible keys round-robin (a fixed order that
// depends on the row's position only), each with an online softmax per map; the CTA joins them, adds the sink to the denominator, and
// finishes the head: differential combination and unit RMS, gate, store.
template <typename TA>
__global__ void __launch_bounds__(128) hy_win_attention_kernel(HyWinAttn a, const TA* __restrict__ q, int ldq, const TA* __restrict__ cache, const float* __restrict__ sink,
                                                               const TA* __restrict__ gate, int ldg, TA* __restrict__ out, int ldo, float eps, HyRows r) {
    HY_PDL();
    extern __shared__ float sm[];
    __shared__ float red[32];
    const int t = blockIdx.x, h = blockIdx.y, D = a.dim, VD = a.vdim, NM = a.maps;
    const int KW = a.kv_heads * NM * D, CW = KW + a.kv_heads * VD, g = h / (a.heads / a.kv_heads);
    float* qs = sm;                              // [NM][D]
    float* part = qs + NM * D;                   // [4][NM][VD]
    float* mm = part + 4 * NM * VD;              // [4][NM]
    float* ll = mm + 4 * NM;                     // [4][NM]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < NM * D; i += blockDim.x) qs[i] = ldf(q + (long long)t * ldq + (long long)h * NM * D + i) * a.scale;
    __syncthreads();
    const int seq = r.row_seq[t], pos = r.positions[t];
    const int32_t* bt = r.block_tables + (long long)seq * r.max_pages_per_seq;
    const WinKeys wk(pos, a.window, a.keep_first);
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, acc[2][WIN_MAXV];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp)
#pragma unroll
        for (int i = 0; i < WIN_MAXV; ++i) acc[mp][i] = 0.f;
    for (int i = warp; i < wk.n; i += 4) {
        const int j = wk.key(i);
        const TA* row = cache + ((long long)bt[j >> 6] * 64 + (j & 63)) * CW;
        const TA* kr = row + (long long)g * NM * D; const TA* vr = row + KW + (long long)g * VD;
        float vv[WIN_MAXV];
#pragma unroll
        for (int c = 0; c < WIN_MAXV; ++c) vv[c] = lane + 32 * c < VD ? ldf(vr + lane + 32 * c) : 0.f;
#pragma unroll
        for (int mp = 0; mp < 2; ++mp) {
            if (mp >= NM) break;
            float d = 0.f;
            for (int c = lane; c < D; c += 32) d = fmaf(qs[mp * D + c], ldf(kr + mp * D + c), d);
            d = warp_sum(d);
            const float mn = fmaxf(m[mp], d), corr = expf(m[mp] - mn), p = expf(d - mn);
            l[mp] = l[mp] * corr + p; m[mp] = mn;
#pragma unroll
            for (int c = 0; c < WIN_MAXV; ++c) acc[mp][c] = fmaf(p, vv[c], acc[mp][c] * corr);
        }
    }
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
        if (mp >= NM) break;
#pragma unroll
        for (int c = 0; c < WIN_MAXV; ++c) if (lane + 32 * c < VD) part[(warp * NM + mp) * VD + lane + 32 * c] = acc[mp][c];
        if (lane == 0) { mm[warp * NM + mp] = m[mp]; ll[warp * NM + mp] = l[mp]; }
    }
    __syncthreads();
    float f[2][4], inv[2];
    for (int mp = 0; mp < NM; ++mp) {
        float M = sink ? sink[h] : -INFINITY, L = 0.f;
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mm[w * NM + mp]);
        for (int w = 0; w < 4; ++w) { f[mp][w] = mm[w * NM + mp] == -INFINITY ? 0.f : expf(mm[w * NM + mp] - M); L = fmaf(f[mp][w], ll[w * NM + mp], L); }
        if (sink) L += expf(sink[h] - M);
        inv[mp] = 1.0f / L;
    }
    float ss = 0.f;
    float o[WIN_MAXV];          // channel threadIdx.x + 128 * i of the head
#pragma unroll
    for (int i = 0; i < WIN_MAXV / 4; ++i) {
        const int c = threadIdx.x + 128 * i; o[i] = 0.f;
        if (c < VD) {
            float a1 = 0.f;
            for (int w = 0; w < 4; ++w) a1 = fmaf(f[0][w], part[(w * NM) * VD + c], a1);
            a1 *= inv[0];
            if (NM == 2) {
                float a2 = 0.f;
                for (int w = 0; w < 4; ++w) a2 = fmaf(f[1][w], part[(w * NM + 1) * VD + c], a2);
                a1 = a1 - a.lambda * (a2 * inv[1]);
            }
            o[i] = a1; ss = fmaf(a1, a1, ss);
        }
    }
    float post = 1.f;
    if (NM == 2) post = a.out_scale / sqrtf(block_sum(ss, red) / (float)VD + eps);
#pragma unroll
    for (int i = 0; i < WIN_MAXV / 4; ++i) {
        const int c = threadIdx.x + 128 * i;
        if (c < VD) {
            float y = o[i] * post;
            if (a.gate == 1) y *= sigmoidf_(ldf(gate + (long long)t * ldg + (long long)h * VD + c));
            else if (a.gate == 2) y *= sigmoidf_(ldf(gate + (long long)t * ldg + h));
            stf(out + (long long)t * ldo + (long long)h * VD + c, y);
        }
    }
}

}  // namespace

cudaError_t hy_rmsnorm_pair(bool f32, const float* x, const int32_t* rows, const float* w1, void* out1, const float* w2, void* out2, int ldo, int T, int W, float eps, cudaStream_t s) {
    if (T <= 0) return cudaSuccess;
    return f32 ? launch_plain(hy_rmsnorm_pair_kernel<float>, dim3(T), dim3(256), 0, s, x, rows, w1, (float*)out1, w2, (float*)out2, ldo, W, eps)
               : launch_plain(hy_rmsnorm_pair_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, s, x, rows, w1, (__nv_bfloat16*)out1, w2, (__nv_bfloat16*)out2, ldo, W, eps);
}

cudaError_t hy_win_prep(bool f32, const HyWinAttn& a, void* q, int ldq, const void* k, const void* v, int ldkv, const float* q_norm_w, const float* k_norm_w, float eps, void* cache,
                        const HyRows& r, cudaStream_t s) {
    if (r.T <= 0 || (!a.qk_norm && !k)) return cudaSuccess;
    using bf = __nv_bfloat16;
    return f32 ? launch_plain(hy_win_prep_kernel<float>, dim3(r.T), dim3(128), 0, s, a, (float*)q, ldq, (const float*)k, (const float*)v, ldkv, q_norm_w, k_norm_w, eps, (float*)cache, r)
               : launch_plain(hy_win_prep_kernel<bf>, dim3(r.T), dim3(128), 0, s, a, (bf*)q, ldq, (const bf*)k, (const bf*)v, ldkv, q_norm_w, k_norm_w, eps, (bf*)cache, r);
}

bool hy_win_supported(const HyWinAttn& a) {
    return a.maps >= 1 && a.maps <= 2 && a.vdim <= 32 * WIN_MAXV && a.dim >= 1 && a.heads % a.kv_heads == 0 &&
           (size_t)(a.maps * a.dim + 4 * a.maps * a.vdim + 8 * a.maps) * 4 <= 200 * 1024;
}

cudaError_t hy_win_attention(bool f32, const HyWinAttn& a, const void* q, int ldq, const void* cache, const float* sink, const void* gate, int ldg, void* out, int ldo, float eps,
                             const HyRows& r, cudaStream_t s) {
    if (r.T <= 0) return cudaSuccess;
    if (!hy_win_supported(a)) return cudaErrorInvalidValue;
    using bf = __nv_bfloat16;
    const size_t smem = (size_t)(a.maps * a.dim + 4 * a.maps * a.vdim + 8 * a.maps) * 4;
    if (smem > 48 * 1024) {
        cudaError_t e = f32 ? cudaFuncSetAttribute(hy_win_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                            : cudaFuncSetAttribute(hy_win_attention_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return f32 ? launch_plain(hy_win_attention_kernel<float>, dim3(r.T, a.heads), dim3(128), smem, s, a, (const float*)q, ldq, (const float*)cache, sink, (const float*)gate, ldg,
                              (float*)out, ldo, eps, r)
               : launch_plain(hy_win_attention_kernel<bf>, dim3(r.T, a.heads), dim3(128), smem, s, a, (const bf*)q, ldq, (const bf*)cache, sink, (const bf*)gate, ldg, (bf*)out, ldo,
                              eps, r);
}

}  // namespace oa
