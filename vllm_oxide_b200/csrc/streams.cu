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
template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
stream_norm_kernel(float* __restrict__ streams, const TY* __restrict__ y, const float* __restrict__ mix,
                   const float* __restrict__ outc, const float* __restrict__ inc, const float* __restrict__ weight,
                   const int* __restrict__ rows, TO* __restrict__ out, int S, int W, int groups, float eps, int copies) {
    pdl_launch_dependents();
    pdl_wait(40);
    extern __shared__ float u_row[];
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
    for (int i = tid; i < W; i += blockDim.x) {
        float old[VOB_MAX_STREAMS], u = 0.f;
#pragma unroll
        for (int s = 0; s < VOB_MAX_STREAMS; ++s) old[s] = s < S ? xs[(size_t)s * W + i] : 0.f;
        if (y) {
            const float yv = ld_f(y + (size_t)src * W + i);
#pragma unroll
            for (int t = 0; t < VOB_MAX_STREAMS; ++t) {
                if (t < S) {
                    float nv = 0.f;
#pragma unroll
                    for (int s = 0; s < VOB_MAX_STREAMS; ++s)
                        if (s < S) nv = fmaf(c_mix[s * S + t], old[s], nv);
                    nv = fmaf(c_out[t], yv, nv);
                    if (!rows) xs[(size_t)t * W + i] = nv;
                    u = fmaf(c_in[t], nv, u);
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < VOB_MAX_STREAMS; ++t)
                if (t < S) u = fmaf(c_in[t], old[t], u);
        }
        u_row[i] = u;
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
        for (int i = tid; i < gw; i += blockDim.x) {
            const float v = weight[g * gw + i] * (part[i] * inv);
            for (int c = 0; c < copies; ++c) st_f(o + (size_t)c * W + g * gw + i, v);
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
#define VOB_SN(TY, TO)                                                                                                     \
    do {                                                                                                                   \
        if (smem > 48 * 1024) {                                                                                            \
            cudaError_t e = cudaFuncSetAttribute(stream_norm_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                           \
        }                                                                                                                  \
        return vob_launch(stream_norm_kernel<TY, TO>, dim3(R), dim3(256), smem, stream, streams, (const TY*)y, mix, outc, inc, weight, \
                          rows, (TO*)out, S, W, groups, eps, copies);                                                      \
    } while (0)
    const int yc = y ? y_code : out_code == VOB_F32 ? VOB_F32 : VOB_BF16;
    if (yc == VOB_F32 && out_code == VOB_F32) VOB_SN(float, float);
    if (yc == VOB_BF16 && out_code == VOB_BF16) VOB_SN(__nv_bfloat16, __nv_bfloat16);
    if (yc == VOB_BF16 && out_code == VOB_F32) VOB_SN(__nv_bfloat16, float);
    if (yc == VOB_F32 && out_code == VOB_BF16) VOB_SN(float, __nv_bfloat16);
#undef VOB_SN
    return VOB_ERR_BAD_ARG;
}
