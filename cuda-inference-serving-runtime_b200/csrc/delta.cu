// The gated delta rule: a recurrent mixer whose state per head is a matrix S [key_dim, value_dim] in float.
//
// Per token and head (query/key head g = head / (heads / kv_heads)), with q and k unit vectors, beta in (0, 1) and
// a decay in (0, 1):
//     S <- decay * S;   u = beta * (v - S^T k);   S <- S + k u^T;   o = S^T q          (o reads this token's write)
//
// Three kernels around the step's one stacked projection proj [T, cols] = h W^T (float):
//   delta_prepare    per token: the short causal convolution over time of the q, k and v channels (taps weights per
//                    channel, the last one the current token's; inputs before the portion come from the request's
//                    kept inputs, zeros before the sequence), silu, unit norm of q and k per head
//                    (x / sqrt(sum x^2 + norm_eps), q times key_dim^-1/2), beta = sigmoid(.), and
//                    decay = exp(-exp(A_log) * softplus(a + dt_bias)).
//   delta_keep       per request: the last taps - 1 convolution inputs become the request's kept inputs.
//   delta_recurrence per (request, head, 8 value columns): one warp walks the portion's tokens in order.  A column of
//                    S evolves on its own, so four lanes share a column (each holds a quarter of its rows in
//                    registers) and the two dot products are finished by two shuffles.  Loads of the next token are
//                    issued before the current token's arithmetic.
//   delta_output     per (token, head): o / sqrt(mean(o^2) + eps) * norm_w * silu(gate), rounded to the operand type of
//                    the output projection.
// A request's row of the state tensor holds [heads][key_dim][value_dim] and then [taps - 1][conv channels], all float.
// A portion of a prompt and a single decoded token take the same path, so a position's result does not depend on
// how the sequence was cut.  Everything that enters the recurrence is float.
#include "common.cuh"

static bool g_pdl = false;
CISR_EXPORT void cisr_delta_set_pdl(int on) { g_pdl = on != 0; }

namespace {
__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// conv channels: [q: kvh * dk][k: kvh * dk][v: heads * dv]; proj columns: the same, then gate [heads * dv], b [heads], a [heads]
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const float* __restrict__ proj, int row_stride, const float* __restrict__ conv_w, int taps,
                     const float* __restrict__ state, long long state_stride, long long keep_offset,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                     const int* __restrict__ token_req, const int* __restrict__ req_slot, const int* __restrict__ q_start,
                     float* __restrict__ qkv, float* __restrict__ beta, float* __restrict__ decay,
                     int heads, int kvh, int dk, int dv, float norm_eps) {
    extern __shared__ float act[];            // conv channels floats
    pdl_trigger();
    const int t = blockIdx.x;
    const int req = token_req[t];
    const int local = t - q_start[req];       // index of the token inside its portion
    const float* keep = state + (size_t)req_slot[req] * state_stride + keep_offset;   // [taps - 1][channels], oldest first
    pdl_wait();
    const int channels = 2 * kvh * dk + heads * dv;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float acc = 0.f;
        for (int j = taps - 1; j >= 0; --j) {             // oldest input first
            const int at = local - j;
            const float x = at >= 0 ? proj[(size_t)(t - j) * row_stride + c] : keep[(size_t)(taps - 1 + at) * channels + c];
            acc = fmaf(conv_w[(size_t)c * taps + (taps - 1 - j)], x, acc);
        }
        act[c] = silu(acc);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    for (int head = warp; head < 2 * kvh; head += n_warps) {          // q heads, then k heads
        float* x = act + head * dk;
        float sq = 0.f;
        for (int d = lane; d < dk; d += 32) sq += x[d] * x[d];
        sq = warp_sum(sq);
        const float inv = (1.f / sqrtf(sq + norm_eps)) * (head < kvh ? 1.f / sqrtf((float)dk) : 1.f);
        for (int d = lane; d < dk; d += 32) x[d] *= inv;
    }
    __syncthreads();
    float* dst = qkv + (size_t)t * channels;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) dst[c] = act[c];
    const float* row = proj + (size_t)t * row_stride;
    const int b_col = channels + heads * dv, a_col = b_col + heads;
    for (int hd = threadIdx.x; hd < heads; hd += blockDim.x) {
        beta[(size_t)t * heads + hd] = 1.f / (1.f + expf(-row[b_col + hd]));
        decay[(size_t)t * heads + hd] = expf(-expf(a_log[hd]) * softplus(row[a_col + hd] + dt_bias[hd]));
    }
}

__global__ void delta_keep_kernel(const float* __restrict__ proj, int row_stride, float* __restrict__ state, long long state_stride,
                                  long long keep_offset, const int* __restrict__ req_slot, const int* __restrict__ q_start,
                                  const int* __restrict__ q_len, int taps, int channels) {
    const int req = blockIdx.x;
    float* keep = state + (size_t)req_slot[req] * state_stride + keep_offset;
    const int n = q_len[req], first = q_start[req], kept = taps - 1;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        // a channel is one thread's: it reads what it needs of the old rows before it overwrites them (rows move towards 0)
        for (int i = 0; i < kept; ++i) {
            const int at = n - kept + i;                  // index in the portion of the input that lands in row i
            keep[(size_t)i * channels + c] = at >= 0 ? proj[(size_t)(first + at) * row_stride + c] : keep[(size_t)(i + n) * channels + c];
        }
    }
}

// R: rows of a column held by one lane (key_dim <= 4 * R); BUFS 2: the next token's operands are fetched into a second
// set of registers before the current token's arithmetic (1 where two sets would not fit the register file)
template <int R, int BUFS>
__global__ void __launch_bounds__(32)
delta_recurrence_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ decay,
                        float* __restrict__ state, long long state_stride, const int* __restrict__ req_slot,
                        const int* __restrict__ q_start, const int* __restrict__ q_len, float* __restrict__ out,
                        int heads, int kvh, int dk, int dv) {
    pdl_trigger();
    const int req = blockIdx.x, head = blockIdx.y;
    const int lane = threadIdx.x, part = lane & 3;
    const int col = blockIdx.z * 8 + (lane >> 2);
    const bool live = col < dv;
    const int g = head / (heads / kvh);
    const int channels = 2 * kvh * dk + heads * dv;
    const int first = q_start[req], n = q_len[req];
    float* S = state + (size_t)req_slot[req] * state_stride + (size_t)head * dk * dv;
    pdl_wait();
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = part + 4 * i;
        s[i] = (live && r < dk) ? S[(size_t)r * dv + col] : 0.f;
    }
    const int q_at = g * dk, k_at = kvh * dk + g * dk, v_at = 2 * kvh * dk + head * dv + (live ? col : 0);
    float kq[BUFS][2 * R], vb[BUFS][3];
    auto fetch = [&](int t, int buf) {
        const float* row = qkv + (size_t)t * channels;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int r = part + 4 * i;
            kq[buf][i] = r < dk ? row[k_at + r] : 0.f;
            kq[buf][R + i] = r < dk ? row[q_at + r] : 0.f;
        }
        vb[buf][0] = row[v_at];
        vb[buf][1] = beta[(size_t)t * heads + head];
        vb[buf][2] = decay[(size_t)t * heads + head];
    };
    if (n > 0) fetch(first, 0);
    for (int i0 = 0; i0 < n; i0 += BUFS) {
#pragma unroll
        for (int b = 0; b < BUFS; ++b) {
            const int i = i0 + b;
            if (i >= n) break;
            if (BUFS == 2 && i + 1 < n) fetch(first + i + 1, b ^ 1);
            const float dec = vb[b][2];
            float ks = 0.f;
#pragma unroll
            for (int j = 0; j < R; ++j) { s[j] *= dec; ks = fmaf(kq[b][j], s[j], ks); }
            ks += __shfl_xor_sync(0xffffffffu, ks, 1);
            ks += __shfl_xor_sync(0xffffffffu, ks, 2);
            const float u = vb[b][1] * (vb[b][0] - ks);
            float o = 0.f;
#pragma unroll
            for (int j = 0; j < R; ++j) { s[j] = fmaf(kq[b][j], u, s[j]); o = fmaf(kq[b][R + j], s[j], o); }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (live && part == 0) out[((size_t)(first + i) * heads + head) * dv + col] = o;
            if (BUFS == 1 && i + 1 < n) fetch(first + i + 1, 0);
        }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = part + 4 * i;
        if (live && r < dk) S[(size_t)r * dv + col] = s[i];
    }
}

template <typename OT>
__global__ void __launch_bounds__(128)
delta_output_kernel(const float* __restrict__ o, const float* __restrict__ proj, int row_stride, int gate_col,
                    const float* __restrict__ norm_w, float eps, OT* __restrict__ out, int out_stride, int heads, int dv, int tokens) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t pair = (size_t)blockIdx.x * 4 + warp;            // (token, head)
    const size_t t = pair / heads;
    const int head = (int)(pair - t * heads);
    if (t >= (size_t)tokens) return;
    const float* src = o + pair * dv;
    float sq = 0.f;
    for (int d = lane; d < dv; d += 32) sq += src[d] * src[d];
    sq = warp_sum(sq);
    const float inv = 1.f / sqrtf(sq / (float)dv + eps);
    const float* gate = proj + t * row_stride + gate_col + head * dv;
    OT* dst = out + t * out_stride + head * dv;
    for (int d = lane; d < dv; d += 32) dst[d] = from_float<OT>(src[d] * inv * norm_w[d] * silu(gate[d]));
}
}  // namespace

CISR_EXPORT int cisr_delta_prepare(const float* proj, int row_stride, const float* conv_w, int taps, const float* state,
                                   long long state_stride, long long keep_offset, const float* a_log, const float* dt_bias,
                                   const int* token_req, const int* req_slot, const int* q_start, float* qkv, float* beta,
                                   float* decay, int heads, int kvh, int dk, int dv, float norm_eps, int tokens, void* stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || kvh <= 0 || heads % kvh || taps < 1) return -2;
    const int channels = 2 * kvh * dk + heads * dv;
    if (row_stride < channels + heads * dv + 2 * heads) return -2;
    const size_t smem = sizeof(float) * (size_t)channels;
    if (smem > 200 * 1024) return -3;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(delta_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    return launch_kernel(delta_prepare_kernel, dim3(tokens), dim3(256), smem, (cudaStream_t)stream, g_pdl, proj, row_stride, conv_w, taps,
                         state, state_stride, keep_offset, a_log, dt_bias, token_req, req_slot, q_start, qkv, beta, decay, heads, kvh,
                         dk, dv, norm_eps);
}

CISR_EXPORT int cisr_delta_keep(const float* proj, int row_stride, float* state, long long state_stride, long long keep_offset,
                                const int* req_slot, const int* q_start, const int* q_len, int taps, int channels, int n_req,
                                void* stream) {
    if (n_req <= 0 || taps <= 1) return 0;
    delta_keep_kernel<<<dim3(n_req, (channels + 255) / 256), 256, 0, (cudaStream_t)stream>>>(proj, row_stride, state, state_stride,
                                                                                           keep_offset, req_slot, q_start, q_len, taps, channels);
    return launch_status();
}

CISR_EXPORT int cisr_delta_max_key_dim() { return 256; }

CISR_EXPORT int cisr_delta_recurrence(const float* qkv, const float* beta, const float* decay, float* state, long long state_stride,
                                      const int* req_slot, const int* q_start, const int* q_len, float* out, int heads, int kvh,
                                      int dk, int dv, int n_req, void* stream) {
    if (n_req <= 0) return 0;
    if (dk <= 0 || dk > 256 || dv <= 0 || heads % kvh) return -2;
    const dim3 grid(n_req, heads, (dv + 7) / 8);
    cudaStream_t s = (cudaStream_t)stream;
#define CISR_DELTA(R, B) return launch_kernel(delta_recurrence_kernel<R, B>, grid, dim3(32), 0, s, g_pdl, qkv, beta, decay, state, state_stride, \
                                           req_slot, q_start, q_len, out, heads, kvh, dk, dv)
    if (dk <= 32) CISR_DELTA(8, 2);
    if (dk <= 64) CISR_DELTA(16, 2);
    if (dk <= 128) CISR_DELTA(32, 2);
    CISR_DELTA(64, 1);
#undef CISR_DELTA
}

CISR_EXPORT int cisr_delta_output(const float* o, const float* proj, int row_stride, int gate_col, const float* norm_w, float eps,
                                  void* out, int out_dtype, int out_stride, int heads, int dv, int tokens, void* stream) {
    if (tokens <= 0) return 0;
    const size_t pairs = (size_t)tokens * heads;
    const dim3 grid((unsigned)((pairs + 3) / 4));
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == CISR_BF16)
        return launch_kernel(delta_output_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, g_pdl, o, proj, row_stride, gate_col, norm_w, eps,
                             (__nv_bfloat16*)out, out_stride, heads, dv, tokens);
    return launch_kernel(delta_output_kernel<float>, grid, dim3(128), 0, s, g_pdl, o, proj, row_stride, gate_col, norm_w, eps,
                         (float*)out, out_stride, heads, dv, tokens);
}
