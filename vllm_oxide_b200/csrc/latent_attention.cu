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
#include <mma.h>
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
        // a warp copies whole keys (one page lookup per key, then consecutive elements)
        for (int kk = warp; kk < n; kk += (int)(blockDim.x >> 5)) {
            const int key = k0 + kk;
            const size_t slot = (size_t)table[key / page_size] * page_size + key % page_size;
            float* dst = tile + kk * W;
            for (int c = lane; c < L; c += 32) dst[c] = ld_f(lat + slot * L + c);
            for (int c = lane; c < R; c += 32) dst[L + c] = ld_f(kr + slot * R + c);
        }
        __syncthreads();
        // four keys at a time: their dot products and reductions are independent chains
        for (int kk = 0; kk < n; kk += 4) {
            float sc[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* kv = tile + min(kk + j, n - 1) * W;
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < NL; ++i) {
                    const int c = lane + 32 * i;
                    if (c < L) a = fmaf(ql[i], kv[c], a);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = lane + 32 * i;
                    if (c < R) a = fmaf(qr[i], kv[L + c], a);
                }
                sc[j] = a;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) sc[j] += __shfl_xor_sync(0xffffffffu, sc[j], o);
            }
            float mn = m;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sc[j] = kk + j < n ? sc[j] * scale : -INFINITY;
                mn = fmaxf(mn, sc[j]);
            }
            const float corr = expf(m - mn);            // exp(-inf) = 0 at the first keys
            float p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) p[j] = expf(sc[j] - mn);
            l = fmaf(l, corr, (p[0] + p[1]) + (p[2] + p[3]));
#pragma unroll
            for (int i = 0; i < NL; ++i) {
                const int c = lane + 32 * i;
                float a = acc[i] * corr;
                if (c < L) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) a = fmaf(p[j], tile[min(kk + j, n - 1) * W + c], a);
                }
                acc[i] = a;
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


// ---------------------------------------------------------------------------------------------
// Prompt portions in bfloat16 on the tensor cores (mma.sync through the wmma interface). A block takes 16
// consecutive tokens of one request and up to 4 heads, two warps per head; a tile of 32 keys ([c | kr], L + R
// wide) is brought into shared memory once for all of them. Per head and key tile: S = Q K^T (float32
// accumulation), the softmax of its 16 rows in float32 with the running maximum and sum in registers, P in
// bfloat16, O += P C with O in shared memory as float32 (rescaled row by row when a maximum moves).
// Needs L and R multiples of 16. Rows are a request's seq_starts[s] + 16 * tile .. ; their positions are
// consecutive, so the tile's last row bounds the keys and every row masks what lies behind its own position.
// ---------------------------------------------------------------------------------------------
#define VOB_LTC_BN 32
#define VOB_LTC_PRE 10        // 16-byte pieces of the next key tile a thread holds ahead (the rest of a tile is copied when it is due)
__global__ void __launch_bounds__(256, 1)
latent_attend_tc_kernel(const float* __restrict__ q_lat, long q_ts, long q_hs, const float* __restrict__ q_rot,
                        const __nv_bfloat16* __restrict__ lat, const __nv_bfloat16* __restrict__ kr, const int* __restrict__ block_tables,
                        int max_pages, const int* __restrict__ seq_starts, const int* __restrict__ positions, int page_size, int H, int L,
                        int R, float scale, __nv_bfloat16* __restrict__ out, long o_ts, long o_hs) {
    using namespace nvcuda;
    constexpr int BN = VOB_LTC_BN;
    pdl_launch_dependents();
    pdl_wait(48);
    // two warps per head: each computes one 16-key half of S, owns eight of the 16 rows in the softmax and half of
    // the latent columns in O += P C. The phases are separated by block barriers that every warp passes.
    const int s = blockIdx.z, HB = blockDim.x >> 6, NW = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hh = warp >> 1, half = warp & 1;
    const int h = blockIdx.y * HB + hh;
    const bool head = h < H;
    const int r0 = seq_starts[s] + blockIdx.x * 16, r1 = seq_starts[s + 1];
    if (r0 >= r1) return;
    const int nrows = min(16, r1 - r0);
    const int D = L + R;
    // leading dimensions with a few elements of padding: rows 512 or 1,024 bytes apart would all fall into the same banks
    const int DP = D + 8, LO = L + 4;
    constexpr int LS = BN + 4, LP = BN + 8;
    extern __shared__ __align__(128) unsigned char ltc_smem[];
    __nv_bfloat16* Kt = reinterpret_cast<__nv_bfloat16*>(ltc_smem);                               // [BN][DP]
    __nv_bfloat16* Q = Kt + (size_t)BN * DP + (size_t)hh * 16 * DP;                                // [16][DP] per head
    float* obase = reinterpret_cast<float*>(Kt + (size_t)BN * DP + (size_t)HB * 16 * DP);
    float* O = obase + (size_t)hh * 16 * LO;                                                       // [16][LO] per head
    float* S = obase + (size_t)HB * 16 * LO + hh * 16 * LS;                                        // [16][LS] per head
    __nv_bfloat16* P = reinterpret_cast<__nv_bfloat16*>(obase + (size_t)HB * 16 * LO + HB * 16 * LS) + hh * 16 * LP;
    for (int e = lane + 32 * half; e < 16 * D; e += 64) {
        const int i = e / D, c = e - i * D;
        float v = 0.f;
        if (head && i < nrows)
            v = c < L ? q_lat[(size_t)(r0 + i) * q_ts + (size_t)h * q_hs + c] : q_rot[((size_t)(r0 + i) * H + h) * R + (c - L)];
        Q[i * DP + c] = __float2bfloat16_rn(v);
    }
    for (int e = lane + 32 * half; e < 16 * LO; e += 64) O[e] = 0.f;
    const int pos0 = positions[r0], pos_hi = pos0 + nrows - 1;
    const int* table = block_tables + (size_t)s * max_pages;
    float m[8], l[8];                   // of rows 8 * half .. 8 * half + 7
#pragma unroll
    for (int i = 0; i < 8; ++i) { m[i] = -INFINITY; l[i] = 0.f; }
    const int lat_chunks = L / 8, kr_chunks = R / 8;            // 16-byte pieces of a key
    const int ntiles = L / 16;
    // The key tile as a list of 16-byte pieces, BN keys x (lat_chunks + kr_chunks) pieces: thread t takes pieces
    // t, t + 256, ... The NEXT tile's pieces are fetched into registers while this tile is worked on.
    const int pieces = lat_chunks + kr_chunks, tile_pieces = BN * pieces;
    const int dp_pieces = DP / 8;                    // a row of Kt in 16-byte pieces (DP is a multiple of 8)
    uint4 nxt[VOB_LTC_PRE];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < VOB_LTC_PRE; ++i) {
            const int x = (int)threadIdx.x + i * (int)blockDim.x;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (x < tile_pieces) {
                const int kk = x / pieces, c = x - kk * pieces;
                const int key = k0 + kk;
                if (key <= pos_hi) {
                    const size_t slot = (size_t)table[key / page_size] * page_size + key % page_size;
                    val = c < lat_chunks ? reinterpret_cast<const uint4*>(lat + slot * L)[c]
                                         : reinterpret_cast<const uint4*>(kr + slot * R)[c - lat_chunks];
                }
            }
            nxt[i] = val;
        }
    };
    fetch(0);
    for (int k0 = 0; k0 <= pos_hi; k0 += BN) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < VOB_LTC_PRE; ++i) {
            const int x = (int)threadIdx.x + i * (int)blockDim.x;
            if (x < tile_pieces) {
                const int kk = x / pieces, c = x - kk * pieces;
                reinterpret_cast<uint4*>(Kt)[(size_t)kk * dp_pieces + c] = nxt[i];
            }
        }
        // what of a tile the registers do not hold (small blocks, wide keys) is copied now
        for (int x = (int)threadIdx.x + VOB_LTC_PRE * (int)blockDim.x; x < tile_pieces; x += (int)blockDim.x) {
            const int kk = x / pieces, c = x - kk * pieces;
            const int key = k0 + kk;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (key <= pos_hi) {
                const size_t slot = (size_t)table[key / page_size] * page_size + key % page_size;
                val = c < lat_chunks ? reinterpret_cast<const uint4*>(lat + slot * L)[c]
                                     : reinterpret_cast<const uint4*>(kr + slot * R)[c - lat_chunks];
            }
            reinterpret_cast<uint4*>(Kt)[(size_t)kk * dp_pieces + c] = val;
        }
        if (k0 + BN <= pos_hi) fetch(k0 + BN);
        __syncthreads();
        if (head) {
            // S = Q K^T, this warp's 16 keys
            wmma::fragment<wmma::accumulator, 16, 16, 16, float> c;
            wmma::fill_fragment(c, 0.f);
            for (int ks = 0; ks < D / 16; ++ks) {
                wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> a;
                wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> b;
                wmma::load_matrix_sync(a, Q + ks * 16, DP);
                wmma::load_matrix_sync(b, Kt + (size_t)half * 16 * DP + ks * 16, DP);
                wmma::mma_sync(c, a, b, c);
            }
            wmma::store_matrix_sync(S + half * 16, c, LS, wmma::mem_row_major);
        }
        __syncthreads();
        if (head) {
            // the softmax of this warp's eight rows, one key per lane
            const int key = k0 + lane;
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
                const int i = 8 * half + ii;
                float sc = S[i * LS + lane] * scale;
                if (i >= nrows || key > pos0 + i) sc = -INFINITY;
                const float mn = fmaxf(m[ii], warp_max(sc));
                const bool none = mn == -INFINITY;
                const float p = none ? 0.f : expf(sc - mn);
                const float corr = none ? 1.f : expf(m[ii] - mn);
                l[ii] = fmaf(l[ii], corr, warp_sum(p));
                m[ii] = mn;
                P[i * LP + lane] = __float2bfloat16_rn(p);
                if (corr != 1.f)
                    for (int c = lane; c < L; c += 32) O[i * LO + c] *= corr;
            }
        }
        __syncthreads();
        if (head) {
            // O += P C, this warp's half of the latent columns
            for (int nt = half; nt < ntiles; nt += 2) {
                wmma::fragment<wmma::accumulator, 16, 16, 16, float> c;
                wmma::load_matrix_sync(c, O + nt * 16, LO, wmma::mem_row_major);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> a;
                    wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::row_major> b;
                    wmma::load_matrix_sync(a, P + ks * 16, LP);
                    wmma::load_matrix_sync(b, Kt + (size_t)ks * 16 * DP + nt * 16, DP);
                    wmma::mma_sync(c, a, b, c);
                }
                wmma::store_matrix_sync(O + nt * 16, c, LO, wmma::mem_row_major);
            }
        }
    }
    __syncthreads();
    if (!head) return;
#pragma unroll
    for (int ii = 0; ii < 8; ++ii) {
        const int i = 8 * half + ii;
        if (i < nrows) {
            const float inv = 1.0f / l[ii];
            __nv_bfloat16* orow = out + (size_t)(r0 + i) * o_ts + (size_t)h * o_hs;
            for (int c = lane; c < L; c += 32) orow[c] = __float2bfloat16_rn(O[i * LO + c] * inv);
        }
    }
}

// Heads a block of the tensor-core kernel takes (0: the sizes do not fit it).
static int ltc_heads(int H, int L, int R) {
    if (L % 16 || R % 16 || L <= 0 || R <= 0) return 0;
    const size_t DP = (size_t)L + R + 8;
    const size_t shared = (size_t)VOB_LTC_BN * DP * 2;
    const size_t per_head = 16 * DP * 2 + 16 * ((size_t)L + 4) * 4 + 16 * (VOB_LTC_BN + 4) * 4 + 16 * (VOB_LTC_BN + 8) * 2;
    if (shared + per_head > 200 * 1024) return 0;
    // as many heads as let two blocks share an SM (one block brings its keys in while the other computes) if that
    // is at least two; else as many as fit one block (a key tile read for a single head is read too often)
    int hb = shared + 2 * per_head > 100 * 1024 ? (int)((200 * 1024 - shared) / per_head) : (int)((100 * 1024 - shared) / per_head);
    hb = hb > 4 ? 4 : hb;
    return hb > H ? H : hb;
}

VOB_EXPORT int vob_latent_attend_tc_supported(int H, int L, int R) { return ltc_heads(H, L, R) > 0 ? 1 : 0; }

// q_lat, q_rot, out and the caches as for vob_latent_attend (bfloat16 caches and out only); seq_starts int32
// [seqs + 1]; max_new: no request brings more rows than this.
VOB_EXPORT int vob_latent_attend_tc(const float* q_lat, long q_ts, long q_hs, const float* q_rot, const void* lat, const void* kr,
                                    const int* block_tables, int max_pages, const int* seq_starts, const int* positions, int page_size,
                                    int seqs, int max_new, int H, int L, int R, float scale, void* out, long o_ts, long o_hs,
                                    cudaStream_t stream) {
    if (seqs <= 0 || max_new <= 0) return 0;
    const int hb = ltc_heads(H, L, R);
    if (hb <= 0) return VOB_ERR_UNSUPPORTED;
    if (page_size <= 0 || max_pages <= 0 || seqs > 65535 || (H + hb - 1) / hb > 65535) return VOB_ERR_BAD_ARG;
    const size_t DP = (size_t)L + R + 8;
    const size_t smem = (size_t)VOB_LTC_BN * DP * 2
        + (size_t)hb * (16 * DP * 2 + 16 * ((size_t)L + 4) * 4 + 16 * (VOB_LTC_BN + 4) * 4 + 16 * (VOB_LTC_BN + 8) * 2);
    cudaError_t e = cudaFuncSetAttribute(latent_attend_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return vob_launch(latent_attend_tc_kernel, dim3((max_new + 15) / 16, (H + hb - 1) / hb, seqs), dim3(64 * hb), smem, stream, q_lat, q_ts,
                      q_hs, q_rot, (const __nv_bfloat16*)lat, (const __nv_bfloat16*)kr, block_tables, max_pages, seq_starts, positions,
                      page_size, H, L, R, scale, (__nv_bfloat16*)out, o_ts, o_hs);
}
