// Several residual streams per token (hyper-connections), and the norm that reads them.
//
// A token carries S streams x_0 .. x_{S-1} of `hidden` floats.  A sub-block reads one mixture of them,
// u = sum_s in[s] x_s, normed; its output y comes back into all streams at once:
// x'_t = sum_s mix[s][t] x_s + out[t] * (y + bias).  One kernel does both ends: it brings the output of the
// sub-block before into the streams (when there is one) and forms the normed input of the next, so the streams
// are read and written once per sub-block and the mixture never exists in memory.
//
//   for row r (source token `src` = rows ? rows[r] : r), channel d:
//     x_s   = source[src][s][d]                       (source_stride 0: all streams read one row, the embedding)
//     x'_t  = y ? sum_s mix[s][t] x_s + out[t] * (y[src][d] + bias[d]) : x_s
//     streams[src][t][d] = x'_t                        (when `store`)
//     u[d]  = sum_t in[t] x'_t                         (in null: plain sum)
//   h[r] = norm(u) * w: layer norm without bias, (u - mean) / sqrt(var + eps) with var the mean squared
//          deviation (kind 0), or u / sqrt(mean(u^2) + eps) (kind 1).
//
// With S = 1, mix = [[1]], out = [1], in = [1] this is the ordinary residual add followed by the norm.
// Everything is float; h is rounded once to its storage type.  Sums run in a fixed order (streams in index
// order, the row's statistics by block_sum), so a row's result does not depend on the batch around it.
#include "common.cuh"

static bool g_pdl = false;
CISR_EXPORT void cisr_hyper_set_pdl(int on) { g_pdl = on != 0; }

namespace {
constexpr int MAX_STREAMS = 16;

// MS: the most streams this instance holds in registers (4, 8 or 16)
template <typename WT, typename OT, int MS>
__global__ void __launch_bounds__(MS == 4 ? 1024 : 256)
hyper_mix_norm_kernel(const float* __restrict__ source, long long source_stride, float* __restrict__ streams,
                      const float* __restrict__ y, const float* __restrict__ bias, const float* __restrict__ mix,
                      const float* __restrict__ out_w, const float* __restrict__ in_w, const WT* __restrict__ norm_w,
                      OT* __restrict__ h, const int* __restrict__ rows, int n_streams, int hidden, float eps, int kind,
                      int store) {
    extern __shared__ float row_cache[];      // hidden floats: the mixture u
    __shared__ float scratch[32];
    __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_out[MAX_STREAMS], s_in[MAX_STREAMS];
    pdl_trigger();
    const int S = n_streams;
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = mix ? mix[i] : ((i / S) == (i % S) ? 1.f : 0.f);
    for (int i = threadIdx.x; i < S; i += blockDim.x) { s_out[i] = out_w ? out_w[i] : 1.f; s_in[i] = in_w ? in_w[i] : 1.f; }
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r);
    pdl_wait();
    __syncthreads();
    const float* xs = source + src * (source_stride ? (size_t)S * hidden : (size_t)hidden);
    float* xd = streams + src * (size_t)S * hidden;
    const float* yr = y ? y + src * hidden : nullptr;
    float sum = 0.f;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
        float x[MS];
#pragma unroll
        for (int s = 0; s < MS; ++s)
            if (s < S) x[s] = xs[(size_t)s * source_stride + d];
        float u = 0.f;
        if (yr) {
            const float yv = yr[d] + (bias ? bias[d] : 0.f);
#pragma unroll
            for (int t = 0; t < MS; ++t) {
                if (t >= S) break;
                float v = 0.f;
#pragma unroll
                for (int s = 0; s < MS; ++s)
                    if (s < S) v = fmaf(s_mix[s * S + t], x[s], v);
                v = fmaf(s_out[t], yv, v);
                if (store) xd[(size_t)t * hidden + d] = v;
                u = fmaf(s_in[t], v, u);
            }
        } else {
#pragma unroll
            for (int t = 0; t < MS; ++t) {
                if (t >= S) break;
                if (store) xd[(size_t)t * hidden + d] = x[t];
                u = fmaf(s_in[t], x[t], u);
            }
        }
        row_cache[d] = u;
        sum += u;
    }
    if (!h) return;
    float mean = 0.f;
    if (kind == 0) mean = block_sum(sum, scratch) / (float)hidden;
    float sq = 0.f;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) { const float c = row_cache[d] - mean; sq += c * c; }
    const float var = block_sum(sq, scratch) / (float)hidden;
    const float inv = 1.f / sqrtf(var + eps);
    OT* o = h + (size_t)r * hidden;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x)
        o[d] = from_float<OT>((row_cache[d] - mean) * inv * to_float(norm_w[d]));
}

// out[t][d] = sum over the streams of token t (the residual stream as one vector: what a probe of a layer's output reads)
__global__ void hyper_sum_kernel(const float* __restrict__ streams, float* __restrict__ out, int n_streams, int hidden) {
    const size_t t = blockIdx.x;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
        float u = 0.f;
        for (int s = 0; s < n_streams; ++s) u += streams[(t * n_streams + s) * hidden + d];
        out[t * hidden + d] = u;
    }
}
}  // namespace

CISR_EXPORT int cisr_hyper_max_streams() { return MAX_STREAMS; }

// source: float [T, S, hidden] (source_is_row = 0) or [T, hidden] read as every stream (1); streams: float [T, S, hidden]
// (may be the same buffer as source); y, bias, mix, out_w, in_w, rows may be null; h null: streams only.
CISR_EXPORT int cisr_hyper_mix_norm(const float* source, int source_is_row, float* streams, const float* y, const float* bias,
                                    const float* mix, const float* out_w, const float* in_w, const void* norm_w, int w_dtype,
                                    void* h, int h_dtype, const int* rows, int n_rows, int n_streams, int hidden, float eps,
                                    int kind, int store, void* stream) {
    if (n_rows <= 0) return 0;
    if (n_streams < 1 || n_streams > MAX_STREAMS || hidden <= 0 || (kind != 0 && kind != 1)) return -2;
    if (h && !norm_w) return -2;
    const size_t smem = sizeof(float) * (size_t)hidden;
    if (smem > 200 * 1024) return -3;
    const long long stride = source_is_row ? 0 : hidden;
    cudaStream_t s = (cudaStream_t)stream;
#define CISR_HYPER_MS(WT, OT, MS)                                                                                       \
    do {                                                                                                                \
        static size_t configured = 48 * 1024;                                                                           \
        if (smem > configured) {                                                                                        \
            cudaError_t e = cudaFuncSetAttribute(hyper_mix_norm_kernel<WT, OT, MS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                        \
            configured = smem;                                                                                          \
        }                                                                                                               \
        /* few rows (a decode step): the row's channels on four times the threads, so that its loads are in flight together */ \
        const int threads = (MS == 4 && n_rows <= 64 && hidden >= 1024) ? 1024 : 256;                                   \
        return launch_kernel(hyper_mix_norm_kernel<WT, OT, MS>, dim3(n_rows), dim3(threads), smem, s, g_pdl, source, stride, streams, y, bias, \
                             mix, out_w, in_w, (const WT*)norm_w, (OT*)h, rows, n_streams, hidden, eps, kind, store);   \
    } while (0)
#define CISR_HYPER(WT, OT)                                                 \
    do {                                                                   \
        if (n_streams <= 4) CISR_HYPER_MS(WT, OT, 4);                      \
        if (n_streams <= 8) CISR_HYPER_MS(WT, OT, 8);                      \
        CISR_HYPER_MS(WT, OT, 16);                                         \
    } while (0)
    if (w_dtype == CISR_BF16 && h_dtype == CISR_BF16) CISR_HYPER(__nv_bfloat16, __nv_bfloat16);
    if (w_dtype == CISR_F32 && h_dtype == CISR_F32) CISR_HYPER(float, float);
    if (w_dtype == CISR_F32 && h_dtype == CISR_BF16) CISR_HYPER(float, __nv_bfloat16);
    CISR_HYPER(__nv_bfloat16, float);
#undef CISR_HYPER
#undef CISR_HYPER_MS
}

CISR_EXPORT int cisr_hyper_sum(const float* streams, float* out, int tokens, int n_streams, int hidden, void* stream) {
    if (tokens <= 0) return 0;
    hyper_sum_kernel<<<tokens, 256, 0, (cudaStream_t)stream>>>(streams, out, n_streams, hidden);
    return launch_status();
}
