// A residual kept as several streams (hyper-connections), and the RMS norm in groups that reads it.
//
// The residual of a token is S vectors x_1 .. x_S of W floats (float32, [T, S, W]). A sublayer reads
// one vector u = sum_s in[s] x_s, normalised; its output y is written back to all streams at once,
//     x_t <- sum_s mix[s, t] x_s + out[t] * y        (mix is indexed [from, to]),
// and that write is not done when y is produced: it is handed on and done by the kernel that reads
// the streams next (one pass over the row instead of two, as the single-stream residual add is
// folded into the next norm). S = 1 with mix = out = in = 1 is the ordinary residual sum.
//
// The norm: the vector is cut into `groups` equal consecutive parts, each divided by its own
// sqrt(mean(part^2) + eps); the whole is multiplied by the weight. One group is the plain RMS norm.
// Everything here is float32 (the residual, the sums, the coefficients); only `y` and `out` have
// the activations' type. One block works on one row and sums in a fixed order, so a row's result
// does not depend on what else is in the batch.
#include "common.cuh"
VOB_PDL_SWITCH(streams)

#define VOB_MAX_STREAMS 8

// out[r, c, :] (c < copies, all equal) = weight * groupnorm(sum_s in[s] x'_s) for row src = rows ? rows[r] : r,
// where x' are the streams after the pending write of y (if y is given). Without a row list the
// updated streams are stored; with one they are left as they were (the rows are only looked at).
// `in` null: every coefficient is 1 (the sum of the streams).
// Launch: one block per output row, 256 threads, W floats of shared memory. Bound: memory.
// Four consecutive elements at a time (the widths are multiples of 4 on this path; see the entry point).
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    __device__ static inline void ld(const float* p, float* v) {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    __device__ static inline void st(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec4<__nv_bfloat16> {
    __device__ static inline void ld(const __nv_bfloat16* p, float* v) {
        const uint2 x = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x), b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    __device__ static inline void st(__nv_bfloat16* p, const float* v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 x;
        x.x = *reinterpret_cast<const unsigned*>(&a);
        x.y = *reinterpret_cast<const unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = x;
    }
};

// VEC = 4: every access takes four consecutive elements (W and W / groups multiples of 4, all rows 16-byte aligned);
// VEC = 1: any width. The arithmetic of an element is the same in both.
template <typename TY, typename TO, int VEC>
__global__ void __launch_bounds__(256)
stream_norm_kernel(float* __restrict__ streams, const TY* __restrict__ y, const float* __restrict__ mix,
                   const float* __restrict__ outc, const float* __restrict__ inc, const float* __restrict__ weight,
                   const int* __restrict__ rows, TO* __restrict__ out, int S, int W, int groups, float eps, int copies) {
    pdl_launch_dependents();
    pdl_wait(40);
    extern __shared__ __align__(16) float u_row[];
    __shared__ float red[8];
    __shared__ float c_mix[VOB_MAX_STREAMS * VOB_MAX_STREAMS], c_out[VOB_MAX_STREAMS], c_in[VOB_MAX_STREAMS];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const int tid = threadIdx.x;
    if (tid < S * S) c_mix[tid] = y ? mix[tid] : 0.f;
    if (tid < S) {
        c_out[tid] = y ? outc[tid] : 0.f;
        c_in[tid] = inc ? inc[tid] : 1.f;
    }
    __syncthreads();
    float* xs = streams + (size_t)src * S * W;
    for (int i = tid * VEC; i < W; i += blockDim.x * VEC) {
        float old[VOB_MAX_STREAMS][VEC], u[VEC], yv[VEC];
#pragma unroll
        for (int s = 0; s < VOB_MAX_STREAMS; ++s) {
            if (s < S) {
                if (VEC == 4) Vec4<float>::ld(xs + (size_t)s * W + i, old[s]);
                else old[s][0] = xs[(size_t)s * W + i];
            }
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) u[e] = 0.f;
        if (y) {
            if (VEC == 4) Vec4<TY>::ld(y + (size_t)src * W + i, yv);
            else yv[0] = ld_f(y + (size_t)src * W + i);
#pragma unroll
            for (int t = 0; t < VOB_MAX_STREAMS; ++t) {
                if (t < S) {
                    float nv[VEC];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        float a = 0.f;
#pragma unroll
                        for (int s = 0; s < VOB_MAX_STREAMS; ++s)
                            if (s < S) a = fmaf(c_mix[s * S + t], old[s][e], a);
                        a = fmaf(c_out[t], yv[e], a);
                        nv[e] = a;
                        u[e] = fmaf(c_in[t], a, u[e]);
                    }
                    if (!rows) {
                        if (VEC == 4) Vec4<float>::st(xs + (size_t)t * W + i, nv);
                        else xs[(size_t)t * W + i] = nv[0];
                    }
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < VOB_MAX_STREAMS; ++t)
                if (t < S) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) u[e] = fmaf(c_in[t], old[t][e], u[e]);
                }
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) u_row[i + e] = u[e];
    }
    __syncthreads();
    const int gw = W / groups;
    const int lane = tid & 31, wid = tid >> 5;
    TO* o = out + (size_t)r * copies * W;
    for (int g = 0; g < groups; ++g) {
        const float* part = u_row + g * gw;
        float ss = 0.f;
        for (int i = tid; i < gw; i += blockDim.x) ss = fmaf(part[i], part[i], ss);
        ss = warp_sum(ss);
        if (lane == 0) red[wid] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int k = 0; k < (int)(blockDim.x >> 5); ++k) tot += red[k];
        const float inv = 1.0f / sqrtf(tot / (float)gw + eps);
        for (int i = tid * VEC; i < gw; i += blockDim.x * VEC) {
            float v[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = weight[g * gw + i + e] * (part[i + e] * inv);
            for (int c = 0; c < copies; ++c) {
                if (VEC == 4) Vec4<TO>::st(o + (size_t)c * W + g * gw + i, v);
                else st_f(o + (size_t)c * W + g * gw + i, v[0]);
            }
        }
        __syncthreads();
    }
}

// streams float32 [T, S, W]; y [T, W] (element code y_code) or null; mix [S, S], outc [S] (needed with y);
// inc [S] or null; weight [W]; rows int32 [R] or null; out [R, copies, W] (element code out_code).
VOB_EXPORT int vob_stream_norm(float* streams, const void* y, int y_code, const float* mix, const float* outc, const float* inc,
                               const float* weight, const int* rows, void* out, int out_code, int R, int S, int W, int groups,
                               float eps, int copies, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (S < 1 || S > VOB_MAX_STREAMS || W <= 0 || groups < 1 || W % groups != 0 || copies < 1) return VOB_ERR_BAD_ARG;
    if (y && (!mix || !outc)) return VOB_ERR_BAD_ARG;
    if ((size_t)W * 4 > 200 * 1024) return VOB_ERR_UNSUPPORTED;
    const size_t smem = (size_t)W * 4;
    // four elements at a time where every row of every operand then starts on 16 bytes
    const bool vec = W % 4 == 0 && (W / groups) % 4 == 0 && (uintptr_t)streams % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)out % 16 == 0;
#define VOB_SN_V(TY, TO, V)                                                                                                \
    do {                                                                                                                   \
        if (smem > 48 * 1024) {                                                                                            \
            cudaError_t e = cudaFuncSetAttribute(stream_norm_kernel<TY, TO, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                           \
        }                                                                                                                  \
        return vob_launch(stream_norm_kernel<TY, TO, V>, dim3(R), dim3(256), smem, stream, streams, (const TY*)y, mix, outc, inc, weight, \
                          rows, (TO*)out, S, W, groups, eps, copies);                                                      \
    } while (0)
#define VOB_SN(TY, TO)                     \
    do {                                   \
        if (vec) VOB_SN_V(TY, TO, 4);      \
        else VOB_SN_V(TY, TO, 1);          \
    } while (0)
    const int yc = y ? y_code : out_code == VOB_F32 ? VOB_F32 : VOB_BF16;
    if (yc == VOB_F32 && out_code == VOB_F32) VOB_SN(float, float);
    if (yc == VOB_BF16 && out_code == VOB_BF16) VOB_SN(__nv_bfloat16, __nv_bfloat16);
    if (yc == VOB_BF16 && out_code == VOB_F32) VOB_SN(__nv_bfloat16, float);
    if (yc == VOB_F32 && out_code == VOB_BF16) VOB_SN(float, __nv_bfloat16);
#undef VOB_SN
#undef VOB_SN_V
    return VOB_ERR_BAD_ARG;
}
