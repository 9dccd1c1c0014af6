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
//   delta_recurrence per (request, head, a few value columns): one warp walks the portion's tokens in order.  A column of
//                    S evolves on its own, so 4 to 32 lanes share a column (each holds its share of the rows in
//                    registers) and the two dot products are finished by shuffles.  The tokens' operands are staged
//                    through shared memory a block of tokens ahead.
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
__global__ void __launch_bounds__(1024)
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

// L lanes share a column of the state and each holds R of its rows in registers (key_dim <= L * R): row r is lane
// r % L's.  A warp owns 32 / L columns.  The walk is a chain of dependent instructions, so a warp runs at a fraction of
// the issue rate whatever else runs beside it; what counts is how few instructions a token costs it.  Eight warps form
// a CTA and share the staged tokens (each thread copies a share of them); the host picks L = 8 unless the launch would
// then have fewer CTAs than the device has SMs.  The tokens' operands come through shared memory in blocks of
// STAGE_TOKENS tokens, two blocks in flight (cp.async), so the walk over the tokens waits for memory once per block and
// not once per token: per token a row [k: dk][q: dk][beta][decay][v: the CTA's columns].
constexpr int STAGE_TOKENS = 16;
constexpr int DELTA_THREADS = 256;            // eight warps share the staged tokens; a CTA owns 256 / L columns of one head
__host__ __device__ inline int stage_stride(int dk, int columns) { return 2 * dk + 2 + columns; }

__device__ __forceinline__ void copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int R, int L>
__global__ void __launch_bounds__(DELTA_THREADS)
delta_recurrence_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ decay,
                        float* __restrict__ state, long long state_stride, const int* __restrict__ req_slot,
                        const int* __restrict__ q_start, const int* __restrict__ q_len, float* __restrict__ out,
                        int heads, int kvh, int dk, int dv) {
    extern __shared__ float stage[];          // [2][STAGE_TOKENS][stage_stride(dk, columns of the CTA)]
    pdl_trigger();
    constexpr int CPC = DELTA_THREADS / L;    // columns per CTA
    const int req = blockIdx.x, head = blockIdx.y;
    const int tid = threadIdx.x, part = tid % L, mine = tid / L;
    const int col0 = blockIdx.z * CPC, col = col0 + mine;
    const bool live = col < dv;
    const int g = head / (heads / kvh);
    const int channels = 2 * kvh * dk + heads * dv;
    const int first = q_start[req], n = q_len[req];
    float* S = state + (size_t)req_slot[req] * state_stride + (size_t)head * dk * dv;
    const int stride = stage_stride(dk, CPC), cols = min(CPC, dv - col0);
    const int q_at = g * dk, k_at = kvh * dk + g * dk, v_at = 2 * kvh * dk + head * dv + col0;
    const int per_token = 2 * dk + cols + 2;  // floats a token brings: k, q, the CTA's columns of v, beta, decay
    pdl_wait();
    auto fetch = [&](int block, float* buf) {          // tokens [block * STAGE_TOKENS, ...) of the portion, by all threads
        const int t0 = block * STAGE_TOKENS, count = min(STAGE_TOKENS, n - t0);
        for (int i = tid; i < count * per_token; i += DELTA_THREADS) {
            const int j = i / per_token, e = i - j * per_token;
            const size_t t = (size_t)(first + t0 + j);
            const float* src;
            int at;
            if (e < dk) { src = qkv + t * channels + k_at + e; at = e; }
            else if (e < 2 * dk) { src = qkv + t * channels + q_at + (e - dk); at = e; }
            else if (e < 2 * dk + cols) { src = qkv + t * channels + v_at + (e - 2 * dk); at = 2 * dk + 2 + (e - 2 * dk); }
            else if (e == 2 * dk + cols) { src = beta + t * heads + head; at = 2 * dk; }
            else { src = decay + t * heads + head; at = 2 * dk + 1; }
            copy4(buf + j * stride + at, src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (n > 0) fetch(0, stage);
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = part + L * i;
        s[i] = (live && r < dk) ? S[(size_t)r * dv + col] : 0.f;
    }
    const int n_blocks = (n + STAGE_TOKENS - 1) / STAGE_TOKENS;
    float o_wait = 0.f;                           // the last token's read-out, not reduced over the column's lanes yet
    int o_token = -1;                             // and its row of `out`
    for (int block = 0; block < n_blocks; ++block) {
        float* buf = stage + (block & 1) * STAGE_TOKENS * stride;
        if (block + 1 < n_blocks) {
            fetch(block + 1, stage + ((block + 1) & 1) * STAGE_TOKENS * stride);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int t0 = block * STAGE_TOKENS, count = min(STAGE_TOKENS, n - t0);
        // A warp issues in order: the read-out's reduction (which nothing of the next token waits for) would hold up the
        // next token's first instructions, and that token's operands would be asked for only then.  So the operands of
        // token j + 1 are read before token j's reductions begin, and the read-out of token j - 1 is reduced beside
        // token j's k . S, shuffle by shuffle.
        float k[R], q[R], bet, dec, v;
        auto read = [&](int j, float* kk, float* qq, float& b, float& d, float& vv) {
            const float* in = buf + j * stride;
            b = in[2 * dk]; d = in[2 * dk + 1];
            vv = live ? in[2 * dk + 2 + mine] : 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const int r = part + L * i;
                kk[i] = r < dk ? in[r] : 0.f;
                qq[i] = r < dk ? in[dk + r] : 0.f;
            }
        };
        read(0, k, q, bet, dec, v);
        for (int j = 0; j < count; ++j) {
            float ks0 = 0.f, ks1 = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                if (i & 1) ks1 = fmaf(k[i], s[i], ks1); else ks0 = fmaf(k[i], s[i], ks0);
            }
            float ks = ks0 + ks1;                 // k . S_old; the decayed state's share is dec times that
            float kn[R], qn[R], betn = 0.f, decn = 0.f, vn = 0.f;
            if (j + 1 < count) read(j + 1, kn, qn, betn, decn, vn);
#pragma unroll
            for (int off = 1; off < L; off <<= 1) {
                ks += __shfl_xor_sync(0xffffffffu, ks, off);
                o_wait += __shfl_xor_sync(0xffffffffu, o_wait, off);
            }
            if (o_token >= 0 && live && part == 0) out[((size_t)o_token * heads + head) * dv + col] = o_wait;
            const float u = bet * (v - dec * ks);
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                s[i] = fmaf(k[i], u, dec * s[i]);
                if (i & 1) o1 = fmaf(q[i], s[i], o1); else o0 = fmaf(q[i], s[i], o0);
            }
            o_wait = o0 + o1;                     // this lane's share of the read-out: reduced beside the next token's k . S
            o_token = first + t0 + j;
#pragma unroll
            for (int i = 0; i < R; ++i) { k[i] = kn[i]; q[i] = qn[i]; }
            bet = betn; dec = decn; v = vn;
        }
        __syncthreads();                          // the block after next is fetched into this buffer
    }
#pragma unroll
    for (int off = 1; off < L; off <<= 1) o_wait += __shfl_xor_sync(0xffffffffu, o_wait, off);
    if (o_token >= 0 && live && part == 0) out[((size_t)o_token * heads + head) * dv + col] = o_wait;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = part + L * i;
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
    const int threads = (tokens <= 64 && channels >= 1024) ? 1024 : 256;      // few tokens (a decode step): a token's channels on more threads
    return launch_kernel(delta_prepare_kernel, dim3(tokens), dim3(threads), smem, (cudaStream_t)stream, g_pdl, proj, row_stride, conv_w, taps,
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
                                      int dk, int dv, int n_req, int lanes_per_column, void* stream) {
    if (n_req <= 0) return 0;
    if (dk <= 0 || dk > 256 || dv <= 0 || heads % kvh) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    // + 256 floats: a lane's row index runs past a short key head's end; such reads are discarded but must stay inside
    const auto smem_for = [dk](int lanes) { return sizeof(float) * (2 * STAGE_TOKENS * (size_t)stage_stride(dk, DELTA_THREADS / lanes) + 256); };
    static int sms = 0;
    if (!sms) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 148;
    }
    // lanes per column: the fewest that give the launch about four warps per SM (or all 32)
    int lanes = 8;
    while (lanes < 32 && (long long)n_req * heads * ((dv * lanes + DELTA_THREADS - 1) / DELTA_THREADS) < sms) lanes *= 2;
    if (lanes_per_column) {                          // the caller's choice (tests)
        if (lanes_per_column != 4 && lanes_per_column != 8 && lanes_per_column != 16 && lanes_per_column != 32) return -2;
        lanes = lanes_per_column;
    }
    while (lanes < 32 && dk > lanes * 64) lanes *= 2;
#define CISR_DELTA(R, L)                                                                                                  \
    do {                                                                                                                  \
        const size_t smem = smem_for(L);                                                                                  \
        static size_t configured = 48 * 1024;                                                                             \
        if (smem > configured) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(delta_recurrence_kernel<R, L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                          \
            configured = smem;                                                                                            \
        }                                                                                                                 \
        return launch_kernel(delta_recurrence_kernel<R, L>, dim3(n_req, heads, (dv * L + DELTA_THREADS - 1) / DELTA_THREADS), dim3(DELTA_THREADS), smem, s, g_pdl, \
                             qkv, beta, decay, state, state_stride, req_slot, q_start, q_len, out, heads, kvh, dk, dv);   \
    } while (0)
    const int rows = (dk + lanes - 1) / lanes;       // per lane
    if (lanes == 4) {
        if (rows <= 8) CISR_DELTA(8, 4);
        if (rows <= 16) CISR_DELTA(16, 4);
        if (rows <= 32) CISR_DELTA(32, 4);
        CISR_DELTA(64, 4);
    }
    if (lanes == 8) {
        if (rows <= 4) CISR_DELTA(4, 8);
        if (rows <= 8) CISR_DELTA(8, 8);
        if (rows <= 16) CISR_DELTA(16, 8);
        CISR_DELTA(32, 8);
    }
    if (lanes == 16) {
        if (rows <= 2) CISR_DELTA(2, 16);
        if (rows <= 4) CISR_DELTA(4, 16);
        if (rows <= 8) CISR_DELTA(8, 16);
        CISR_DELTA(16, 16);
    }
    if (rows <= 2) CISR_DELTA(2, 32);
    if (rows <= 4) CISR_DELTA(4, 32);
    CISR_DELTA(8, 32);
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
