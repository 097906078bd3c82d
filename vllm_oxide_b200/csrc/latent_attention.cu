// Attention over a latent cache: per token the pages hold ONE latent vector c (width L, shared by
// all heads, already normalised) and ONE rotated key part (width R, shared by all heads), not
// keys and values per head. A head's key is [W_uk c | rotated part] and its value W_uv c, but
// neither is ever built: with q_lat = W_uk^T q_plain (done by the caller as a matrix product)
//     score(i, j) = (q_lat_i . c_j + q_rot_i . kr_j) * scale,   out_lat_i = sum_j softmax_j(score) c_j
// and the caller applies W_uv to out_lat. Causal: row i of a request sees the keys 0 .. position(i)
// of that request, all read from the pages (the step's own tokens were written first).
//
// vob_latent_prep: per token, c = weight * x / sqrt(mean(x^2) + eps) of the first L columns of the
// down projection and the rotary positions on its last R columns, both written to the token's cache
// slot; the rotated query part of every head to a float32 buffer.
// vob_latent_attend: scores, softmax weights and the weighted sum in float32, keys in page order
// from the first, in tiles staged in shared memory; one warp per head, a block takes up to 8 heads
// of one row, so a key tile is read once for all of them. The order of every sum depends only on the row's
// position, never on how the request was cut into steps or on the batch around it. Steps of few rows
// (single tokens) share a row's keys over `splits` blocks, whose partial results a second small kernel
// puts together in a fixed order.
#include "common.cuh"
#include <math.h>
VOB_PDL_SWITCH(latent_attention)

// proj [T, ld]: the query of head h at columns q_off + h * (D + R) (D plain features, then R to be
// rotated); the down projection at columns down_off .. + L + R. lat [pages, 1, page, L], kr [pages,
// 1, page, R] in the cache's type TC. q_rot float32 [T, H, R]. Rows with position < 0 write nothing
// (their q_rot is zero); a slot < 0 writes no cache.
// Launch: one block of 128 threads per token.
template <typename T, typename TC>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T* __restrict__ proj, long ld, int q_off, int H, int D, int R, int down_off, int L,
                   const float* __restrict__ norm_w, float eps, const int* __restrict__ positions, const int* __restrict__ slots,
                   const float* __restrict__ inv_freq, TC* __restrict__ lat, TC* __restrict__ kr, float* __restrict__ q_rot) {
    pdl_launch_dependents();
    pdl_wait(45);
    __shared__ float red[4];
    const int t = blockIdx.x, tid = threadIdx.x;
    const int pos = positions[t];
    const T* row = proj + (size_t)t * ld;
    const int half = R >> 1;
    float* qo = q_rot + (size_t)t * H * R;
    for (int e = tid; e < H * R; e += blockDim.x) {
        float v = 0.f;
        if (pos >= 0) {
            const int h = e / R, f = e - h * R;
            const int i = f < half ? f : f - half;
            const float ang = (float)pos * inv_freq[i];
            const float cs = cosf(ang), sn = sinf(ang);
            const T* qh = row + q_off + (size_t)h * (D + R) + D;
            const float a = ld_f(qh + i), b = ld_f(qh + i + half);
            v = f < half ? a * cs - b * sn : b * cs + a * sn;
        }
        qo[e] = v;
    }
    const int slot = slots ? slots[t] : -1;
    if (pos < 0 || slot < 0) return;
    const T* down = row + down_off;
    float ss = 0.f;
    for (int i = tid; i < L; i += blockDim.x) {
        const float x = ld_f(down + i);
        ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    const float inv = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)L + eps);
    TC* lo = lat + (size_t)slot * L;
    for (int i = tid; i < L; i += blockDim.x) st_f(lo + i, norm_w[i] * (ld_f(down + i) * inv));
    TC* ko = kr + (size_t)slot * R;
    for (int f = tid; f < R; f += blockDim.x) {
        const int i = f < half ? f : f - half;
        const float ang = (float)pos * inv_freq[i];
        const float cs = cosf(ang), sn = sinf(ang);
        const float a = ld_f(down + L + i), b = ld_f(down + L + i + half);
        st_f(ko + f, f < half ? a * cs - b * sn : b * cs + a * sn);
    }
}

VOB_EXPORT int vob_latent_prep(const void* proj, int code, long ld, int q_off, int H, int D, int R, int down_off, int L,
                               const float* norm_w, float eps, const int* positions, const int* slots, const float* inv_freq,
                               void* lat, void* kr, int cache_code, float* q_rot, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || D < 0 || R <= 0 || (R & 1) || L <= 0 || code != cache_code) return VOB_ERR_BAD_ARG;
    VOB_DISPATCH_ELEM(code, return vob_launch(latent_prep_kernel<ElemT, ElemT>, dim3(T), dim3(128), 0, stream, (const ElemT*)proj, ld,
                                              q_off, H, D, R, down_off, L, norm_w, eps, positions, slots, inv_freq, (ElemT*)lat,
                                              (ElemT*)kr, q_rot));
    return 0;
}

// q_lat float32, element (t, h, i) at t * q_ts + h * q_hs + i; q_rot float32 [T, H, R]; out_lat of type
// TO, element (t, h, i) at t * o_ts + h * o_hs + i. NL = ceil(L / 32) registers per lane for q_lat and
// for the weighted sum. Grid (rows, ceil(H / warps)); a block has `warps` warps, one head each.
template <int NL, typename TC, typename TO>
__global__ void __launch_bounds__(256, 1)
latent_attend_kernel(const float* __restrict__ q_lat, long q_ts, long q_hs, const float* __restrict__ q_rot,
                     const TC* __restrict__ lat, const TC* __restrict__ kr, const int* __restrict__ block_tables, int max_pages,
                     const int* __restrict__ row_seq, const int* __restrict__ positions, int page_size, int H, int L, int R,
                     float scale, int KT, TO* __restrict__ out, long o_ts, long o_hs, int splits, float* __restrict__ part) {
    pdl_launch_dependents();
    pdl_wait(46);
    extern __shared__ float tile[];                 // [KT][L + R]
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * (blockDim.x >> 5) + warp;
    const bool head = h < H;
    const int pos = positions[t];
    TO* orow = out + (size_t)t * o_ts + (size_t)(head ? h : 0) * o_hs;
    // with splits > 1 block z takes the z-th share of the row's keys and leaves (max, sum, weighted sum) in `part`
    // [T, H, splits, L + 2]; the shares depend on the row's position and `splits` only
    float* prow = part + (((size_t)t * H + (head ? h : 0)) * splits + blockIdx.z) * (L + 2);
    if (pos < 0) {
        if (head && splits == 1)
            for (int i = lane; i < L; i += 32) st_f(orow + i, 0.f);
        if (head && splits > 1 && lane == 0) { prow[0] = -INFINITY; prow[1] = 0.f; }
        return;
    }
    const int* table = block_tables + (size_t)row_seq[t] * max_pages;
    const int W = L + R;
    float ql[NL], qr[4], acc[NL];
#pragma unroll
    for (int i = 0; i < NL; ++i) {
        const int c = lane + 32 * i;
        ql[i] = (head && c < L) ? q_lat[(size_t)t * q_ts + (size_t)h * q_hs + c] : 0.f;
        acc[i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = lane + 32 * i;
        qr[i] = (head && c < R) ? q_rot[((size_t)t * H + h) * R + c] : 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int share = ((pos + splits) / splits + KT - 1) / KT * KT;      // keys per block, whole tiles
    const int nkeys = min(pos + 1, (int)(blockIdx.z + 1) * share);
    for (int k0 = blockIdx.z * share; k0 < nkeys; k0 += KT) {
        const int n = min(KT, nkeys - k0);
        __syncthreads();
        for (int e = threadIdx.x; e < n * W; e += blockDim.x) {
            const int kk = e / W, c = e - kk * W;
            const int key = k0 + kk;
            const size_t slot = (size_t)table[key / page_size] * page_size + key % page_size;
            tile[e] = c < L ? ld_f(lat + slot * L + c) : ld_f(kr + slot * R + (c - L));
        }
        __syncthreads();
        for (int kk = 0; kk < n; ++kk) {
            const float* kv = tile + kk * W;
            float sc = 0.f;
#pragma unroll
            for (int i = 0; i < NL; ++i) {
                const int c = lane + 32 * i;
                if (c < L) sc = fmaf(ql[i], kv[c], sc);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = lane + 32 * i;
                if (c < R) sc = fmaf(qr[i], kv[L + c], sc);
            }
            sc = warp_sum(sc) * scale;
            const float mn = fmaxf(m, sc);
            const float corr = expf(m - mn);            // exp(-inf) = 0 at the first key
            const float p = expf(sc - mn);
            l = fmaf(l, corr, p);
#pragma unroll
            for (int i = 0; i < NL; ++i) {
                const int c = lane + 32 * i;
                acc[i] = fmaf(p, c < L ? kv[c] : 0.f, acc[i] * corr);
            }
            m = mn;
        }
    }
    if (head && splits == 1) {
        const float inv = 1.0f / l;
#pragma unroll
        for (int i = 0; i < NL; ++i) {
            const int c = lane + 32 * i;
            if (c < L) st_f(orow + c, acc[i] * inv);
        }
    }
    if (head && splits > 1) {
        if (lane == 0) { prow[0] = m; prow[1] = l; }
#pragma unroll
        for (int i = 0; i < NL; ++i) {
            const int c = lane + 32 * i;
            if (c < L) prow[2 + c] = acc[i];
        }
    }
}

// The shares of a row's keys put together, in share order: out = sum_z acc_z e^(m_z - M) / sum_z l_z e^(m_z - M).
// Launch: one warp per (row, head).
template <typename TO>
__global__ void __launch_bounds__(32)
latent_merge_kernel(const float* __restrict__ part, const int* __restrict__ positions, int H, int L, int splits,
                    TO* __restrict__ out, long o_ts, long o_hs) {
    pdl_launch_dependents();
    pdl_wait(47);
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    TO* orow = out + (size_t)t * o_ts + (size_t)h * o_hs;
    const float* p = part + ((size_t)t * H + h) * splits * (L + 2);
    if (positions[t] < 0) {
        for (int i = lane; i < L; i += 32) st_f(orow + i, 0.f);
        return;
    }
    float M = -INFINITY;
    for (int z = 0; z < splits; ++z) M = fmaxf(M, p[(size_t)z * (L + 2)]);
    float l = 0.f;
    for (int z = 0; z < splits; ++z) l = fmaf(p[(size_t)z * (L + 2) + 1], expf(p[(size_t)z * (L + 2)] - M), l);
    const float inv = 1.0f / l;
    for (int i = lane; i < L; i += 32) {
        float a = 0.f;
        for (int z = 0; z < splits; ++z) {
            const float* pz = p + (size_t)z * (L + 2);
            if (pz[1] > 0.f) a = fmaf(pz[2 + i], expf(pz[0] - M), a);
        }
        st_f(orow + i, a * inv);
    }
}

VOB_EXPORT int vob_latent_attend(const float* q_lat, long q_ts, long q_hs, const float* q_rot, const void* lat, const void* kr,
                                 int cache_code, const int* block_tables, int max_pages, const int* row_seq, const int* positions,
                                 int page_size, int T, int H, int L, int R, float scale, void* out, int out_code, long o_ts, long o_hs,
                                 int splits, float* part, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || L <= 0 || R <= 0 || page_size <= 0 || max_pages <= 0 || cache_code != out_code) return VOB_ERR_BAD_ARG;
    if (splits < 1 || splits > 65535 || (splits > 1 && !part) || H > 65535) return VOB_ERR_BAD_ARG;
    if (L > 1024 || R > 128) return VOB_ERR_UNSUPPORTED;
    const int warps = H < 8 ? H : 8;
    const int W = L + R;
    int KT = (int)(40 * 1024 / ((size_t)W * 4));
    KT = KT > 32 ? 32 : KT < 1 ? 1 : KT;
    const size_t smem = (size_t)KT * W * 4;
    dim3 grid(T, (H + warps - 1) / warps, splits), block(32 * warps);
    const int nl = (L + 31) / 32;
    int status = VOB_ERR_BAD_ARG;
#define VOB_LA(N, TC)                                                                                                          \
    status = vob_launch(latent_attend_kernel<N, TC, TC>, grid, block, smem, stream, q_lat, q_ts, q_hs, q_rot, (const TC*)lat, \
                        (const TC*)kr, block_tables, max_pages, row_seq, positions, page_size, H, L, R, scale, KT, (TC*)out, o_ts, o_hs, \
                        splits, part)
#define VOB_LA_N(TC)                       \
    do {                                   \
        if (nl <= 4) { VOB_LA(4, TC); }        \
        else if (nl <= 8) { VOB_LA(8, TC); }   \
        else if (nl <= 16) { VOB_LA(16, TC); } \
        else { VOB_LA(32, TC); }               \
        if (status == 0 && splits > 1)         \
            status = vob_launch(latent_merge_kernel<TC>, dim3(T, H), dim3(32), 0, stream, (const float*)part, positions, H, L, splits, \
                                (TC*)out, o_ts, o_hs);                                                                          \
    } while (0)
    if (cache_code == VOB_F32) VOB_LA_N(float);
    else if (cache_code == VOB_BF16) VOB_LA_N(__nv_bfloat16);
#undef VOB_LA_N
#undef VOB_LA
    return status;
}
