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

__device__ __forceinline__ void copy16(float* dst, const float* src) {      // both 16-byte aligned
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_done() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int R, int L>
__global__ void __launch_bounds__(DELTA_THREADS)
delta_recurrence_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ decay,
                        float* __restrict__ state, long long state_stride, const int* __restrict__ req_slot,
                        const int* __restrict__ q_start, const int* __restrict__ q_len, float* __restrict__ out,
                        int heads, int kvh, int dk, int dv, int below) {
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
    pdl_wait();                               // also where nothing is left to do: the kernel after this one relies on the chain of waits
    if (below > 0 && n >= below) return;      // a portion that long is the chunk kernels'
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

// ------------------------------------------------------------------ the same recurrence, a chunk of tokens at a time
// For the C tokens of a chunk with the state S0 before it, c_t the product of the decays up to token t inside the chunk:
//     S_t = c_t S0 + sum_{i<=t} (c_t / c_i) k_i u_i^T,      u_t + sum_{i<t} A[t][i] u_i = beta_t (v_t - c_t S0^T k_t),
//     A[t][i] = beta_t (c_t / c_i) (k_t . k_i)              (i < t)
// so with T = (I + A)^-1 (lower triangular, ones on the diagonal) and P[t][i] = (c_t / c_i) (q_t . k_i) (i <= t):
//     U = T B,   B[t] = beta_t (v_t - c_t (K S0)[t]);   O[t] = c_t (Q S0)[t] + (P U)[t];   S_C = c_C S0 + sum_i (c_C / c_i) k_i u_i^T.
// T and P depend on no state: `delta_chunk_tables` makes them for every chunk of the step at once, a CTA per (chunk, key head).
// `delta_chunk_walk` then carries the state from chunk to chunk, a CTA per (request, head, 16 or 8 value columns), with
// small matrix products in shared memory instead of a chain of shuffles per token.  Ratios of decays are taken as
// exp(l_t - l_i) from sums of logarithms (t >= i: never above one; a decay of zero is floored at e^-80).  Float throughout.
constexpr int CHUNK = 64, CHUNK_THREADS = 256;
__host__ __device__ inline int chunk_row_stride(int dk) { return dk % 4 == 0 ? dk + 4 : dk + 1; }

__global__ void __launch_bounds__(CHUNK_THREADS)
delta_chunk_tables_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ decay,
                          const int* __restrict__ chunk_req, const int* __restrict__ chunk_t0, const int* __restrict__ q_start,
                          const int* __restrict__ q_len, float* __restrict__ tables, int heads, int kvh, int dk, int dv,
                          int heads_per_cta) {
    // A CTA per (chunk, `heads_per_cta` heads of one key head): the products k_t . k_i and q_t . k_i are the same for every
    // head of a group and are made once per CTA (4 x 4 tiles per thread, tiles above the diagonal skipped); then, head by
    // head, the decays and beta turn them into A and P, and A is inverted.  The host gives a CTA the whole group when the
    // launch has CTAs to spare, and one head when it has not (the heads' turns in a CTA run one after the other).
    extern __shared__ float sm[];
    const int ld = dk + 1, lc_ = CHUNK + 1;
    float* Ks = sm;                           // [CHUNK][dk + 1]
    float* Qs = Ks + CHUNK * ld;              // [CHUNK][dk + 1]
    float* Gk = Qs + CHUNK * ld;              // [CHUNK][CHUNK + 1]: k_t . k_i
    float* Gq = Gk + CHUNK * lc_;             // [CHUNK][CHUNK + 1]: q_t . k_i
    float* As = Gq + CHUNK * lc_;             // [CHUNK][CHUNK + 1]
    float* Ts = As + CHUNK * lc_;             // [CHUNK][CHUNK + 1]
    float* lg = Ts + CHUNK * lc_;             // [CHUNK] sums of log decays
    float* bt = lg + CHUNK;                   // [CHUNK] beta
    pdl_trigger();
    const int chunk = blockIdx.x, head0 = blockIdx.y * heads_per_cta, tid = threadIdx.x;
    const int req = chunk_req[chunk], t0 = chunk_t0[chunk];
    const int count = min(CHUNK, q_len[req] - t0), first = q_start[req] + t0;
    const int g = head0 / (heads / kvh), channels = 2 * kvh * dk + heads * dv;
    pdl_wait();
    {
        const int t = tid >> 2;
        const float* row = qkv + (size_t)(first + t) * channels;
        for (int r = tid & 3; r < dk; r += 4) {
            Ks[t * ld + r] = t < count ? row[kvh * dk + g * dk + r] : 0.f;
            Qs[t * ld + r] = t < count ? row[g * dk + r] : 0.f;
        }
    }
    __syncthreads();
    {
        const int t4 = (tid >> 4) * 4, i4 = (tid & 15) * 4;
        float kk[4][4], qk[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) { kk[a][b] = 0.f; qk[a][b] = 0.f; }
        if (i4 <= t4) {
#pragma unroll 2
            for (int r = 0; r < dk; ++r) {
                float kt[4], qt[4], ki[4];
#pragma unroll
                for (int a = 0; a < 4; ++a) { kt[a] = Ks[(t4 + a) * ld + r]; qt[a] = Qs[(t4 + a) * ld + r]; ki[a] = Ks[(i4 + a) * ld + r]; }
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b) { kk[a][b] = fmaf(kt[a], ki[b], kk[a][b]); qk[a][b] = fmaf(qt[a], ki[b], qk[a][b]); }
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) { Gk[(t4 + a) * lc_ + i4 + b] = kk[a][b]; Gq[(t4 + a) * lc_ + i4 + b] = qk[a][b]; }
    }
    for (int hd = 0; hd < heads_per_cta; ++hd) {
        const int head = head0 + hd;
        float* out_T = tables + ((size_t)chunk * heads + head) * (2 * CHUNK * CHUNK + CHUNK);
        float* out_P = out_T + CHUNK * CHUNK;
        __syncthreads();                      // the products are whole; the head before is done with A, T, lg
        if (tid < CHUNK) {
            bt[tid] = tid < count ? beta[(size_t)(first + tid) * heads + head] : 0.f;
            lg[tid] = tid < count ? fmaxf(logf(decay[(size_t)(first + tid) * heads + head]), -80.f) : 0.f;
        }
        __syncthreads();
        if (tid == 0) {                       // the running sum, in token order
            float sum = 0.f;
            for (int t = 0; t < CHUNK; ++t) { sum += lg[t]; lg[t] = sum; }
        }
        __syncthreads();
        {
            const int t = tid >> 2, i0 = (tid & 3) * 16;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int i = i0 + j;
                const float ratio = i <= t ? expf(lg[t] - lg[i]) : 0.f;
                As[t * lc_ + i] = i < t ? bt[t] * ratio * Gk[t * lc_ + i] : 0.f;
                out_P[t * CHUNK + i] = ratio * Gq[t * lc_ + i];
            }
        }
        if (tid < CHUNK) out_T[2 * CHUNK * CHUNK + tid] = lg[tid];
        __syncthreads();
        // T = (I + A)^-1 by forward substitution: T[t][c] = [t == c] - sum_{c <= i < t} A[t][i] T[i][c].  Four neighbouring
        // lanes own column c and take every fourth i; a row is finished by two shuffles before the next row reads it.
        {
            const int c = tid >> 2, p = tid & 3;
            for (int t = 0; t < CHUNK; ++t) {
                float a = 0.f;
#pragma unroll 4
                for (int i = c + p; i < t; i += 4) a = fmaf(-As[t * lc_ + i], Ts[i * lc_ + c], a);
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                a += __shfl_xor_sync(0xffffffffu, a, 2);
                if (p == 0) Ts[t * lc_ + c] = t < c ? 0.f : (t == c ? 1.f : 0.f) + a;
                __syncwarp();
            }
        }
        __syncthreads();
        {
            const int t = tid >> 2, i0 = (tid & 3) * 16;
#pragma unroll
            for (int j = 0; j < 16; ++j) out_T[t * CHUNK + i0 + j] = Ts[t * lc_ + i0 + j];
        }
    }
}

// COLS value columns per CTA (16, or 8 where that many CTAs would not fill the device): 64 rows x COLS / 4 threads
template <int COLS>
__global__ void __launch_bounds__(CHUNK * COLS / 4)
delta_chunk_walk_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ tables,
                        const int* __restrict__ req_chunk0, float* __restrict__ state, long long state_stride,
                        const int* __restrict__ req_slot, const int* __restrict__ q_start, const int* __restrict__ q_len,
                        float* __restrict__ out, int heads, int kvh, int dk, int dv, int least) {
    extern __shared__ __align__(16) float sm[];
    // Row strides that are multiples of 4 (16-byte rows for vector copies) and 4 mod 32 (rows t, t + 1, ... of a warp's
    // eight fall into different banks); odd key widths keep scalar copies and a stride of dk + 1.
    const bool vec = dk % 4 == 0 && dv % 4 == 0;
    const int ld = chunk_row_stride(dk), lc_ = CHUNK + 4;
    float* Ks = sm;                           // [CHUNK][ld]
    float* Qs = Ks + CHUNK * ld;              // [CHUNK][ld]
    float* Ts = Qs + CHUNK * ld;              // [CHUNK][CHUNK + 4]
    float* Ps = Ts + CHUNK * lc_;             // [CHUNK][CHUNK + 4]
    float* S0 = Ps + CHUNK * lc_;             // [dk][COLS]
    float* Bs = S0 + dk * COLS;         // [CHUNK][COLS]: B, then U
    float* Vs = Bs + CHUNK * COLS;      // [CHUNK][COLS]
    float* lg = Vs + CHUNK * COLS;      // [CHUNK]
    float* bt = lg + CHUNK;                   // [CHUNK]
    float* wl = bt + CHUNK;                   // [CHUNK]: c_C / c_i
    pdl_trigger();
    constexpr int PARTS = COLS / 4, THREADS = CHUNK * PARTS;      // threads per row, threads per CTA
    const int req = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int n = q_len[req];
    const int col0 = blockIdx.z * COLS, cols = min(COLS, dv - col0);
    const int g = head / (heads / kvh), channels = 2 * kvh * dk + heads * dv;
    const int first = q_start[req];
    float* S = state + (size_t)req_slot[req] * state_stride + (size_t)head * dk * dv;
    pdl_wait();
    if (n < least) return;                    // short portions and single tokens are the token-by-token kernel's
    for (int i = tid; i < dk * COLS; i += THREADS) {
        const int r = i / COLS, j = i - r * COLS;
        S0[i] = j < cols ? S[(size_t)r * dv + col0 + j] : 0.f;
    }
    const int t = tid / PARTS, j0 = (tid % PARTS) * 4;     // this thread's four entries of every [CHUNK][COLS] product
    const int n_chunks = (n + CHUNK - 1) / CHUNK;
    for (int c = 0; c < n_chunks; ++c) {
        const int t0 = c * CHUNK, count = min(CHUNK, n - t0);
        const float* tab = tables + ((size_t)(req_chunk0[req] + c) * heads + head) * (2 * CHUNK * CHUNK + CHUNK);
        __syncthreads();                      // the chunk before is done with the buffers (and S0 is whole)
        {   // row t of every operand by the four threads that own row t of the products: all copies are in flight together
            const int part = tid % PARTS;
            const float* row = qkv + (size_t)(first + t0 + t) * channels;
            const bool in = t < count;
            if (vec) {
                const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
                const float* k4 = row + kvh * dk + g * dk;
                const float* q4 = row + g * dk;
                for (int r4 = part; r4 < dk / 4; r4 += PARTS) {
                    if (in) { copy16(Ks + t * ld + 4 * r4, k4 + 4 * r4); copy16(Qs + t * ld + 4 * r4, q4 + 4 * r4); }
                    else { *reinterpret_cast<float4*>(Ks + t * ld + 4 * r4) = zero; *reinterpret_cast<float4*>(Qs + t * ld + 4 * r4) = zero; }
                }
                // dv % 4 == 0: a group of four columns is whole or beyond the head
                if (in && 4 * part < cols) copy16(Vs + t * COLS + 4 * part, row + 2 * kvh * dk + head * dv + col0 + 4 * part);
                else *reinterpret_cast<float4*>(Vs + t * COLS + 4 * part) = zero;
            } else {
                for (int r = part; r < dk; r += PARTS) {
                    Ks[t * ld + r] = in ? row[kvh * dk + g * dk + r] : 0.f;
                    Qs[t * ld + r] = in ? row[g * dk + r] : 0.f;
                }
                for (int j = 4 * part; j < 4 * part + 4; ++j)
                    Vs[t * COLS + j] = (in && j < cols) ? row[2 * kvh * dk + head * dv + col0 + j] : 0.f;
            }
#pragma unroll
            for (int k = part; k < CHUNK / 4; k += PARTS) {
                copy16(Ts + t * lc_ + 4 * k, tab + t * CHUNK + 4 * k);
                copy16(Ps + t * lc_ + 4 * k, tab + CHUNK * CHUNK + t * CHUNK + 4 * k);
            }
        }
        if (tid < CHUNK) {
            const float l = tab[2 * CHUNK * CHUNK + tid];
            lg[tid] = l;
            wl[tid] = expf(tab[2 * CHUNK * CHUNK + CHUNK - 1] - l);
            bt[tid] = tid < count ? beta[(size_t)(first + t0 + tid) * heads + head] : 0.f;
        }
        copies_done();
        __syncthreads();
        // K S0 and Q S0, four columns of row t
        float ks[4] = {0.f, 0.f, 0.f, 0.f}, qs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int r = 0; r < dk; ++r) {
            const float kt = Ks[t * ld + r], qt = Qs[t * ld + r];
            const float4 s4 = *reinterpret_cast<const float4*>(S0 + r * COLS + j0);
            ks[0] = fmaf(kt, s4.x, ks[0]); ks[1] = fmaf(kt, s4.y, ks[1]); ks[2] = fmaf(kt, s4.z, ks[2]); ks[3] = fmaf(kt, s4.w, ks[3]);
            qs[0] = fmaf(qt, s4.x, qs[0]); qs[1] = fmaf(qt, s4.y, qs[1]); qs[2] = fmaf(qt, s4.z, qs[2]); qs[3] = fmaf(qt, s4.w, qs[3]);
        }
        const float ct = expf(lg[t]);
        {
            const float4 v4 = *reinterpret_cast<const float4*>(Vs + t * COLS + j0);
            const float b = bt[t];
            *reinterpret_cast<float4*>(Bs + t * COLS + j0) =
                make_float4(b * (v4.x - ct * ks[0]), b * (v4.y - ct * ks[1]), b * (v4.z - ct * ks[2]), b * (v4.w - ct * ks[3]));
        }
        __syncthreads();
        // U = T B (row t needs rows 0 .. t of B)
        float u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int i = 0; i <= t; ++i) {
            const float w = Ts[t * lc_ + i];
            const float4 b4 = *reinterpret_cast<const float4*>(Bs + i * COLS + j0);
            u[0] = fmaf(w, b4.x, u[0]); u[1] = fmaf(w, b4.y, u[1]); u[2] = fmaf(w, b4.z, u[2]); u[3] = fmaf(w, b4.w, u[3]);
        }
        __syncthreads();                      // every row of B has been read
        *reinterpret_cast<float4*>(Bs + t * COLS + j0) = make_float4(u[0], u[1], u[2], u[3]);
        __syncthreads();
        // O = c_t Q S0 + P U
        float o[4] = {ct * qs[0], ct * qs[1], ct * qs[2], ct * qs[3]};
#pragma unroll 4
        for (int i = 0; i <= t; ++i) {
            const float w = Ps[t * lc_ + i];
            const float4 u4 = *reinterpret_cast<const float4*>(Bs + i * COLS + j0);
            o[0] = fmaf(w, u4.x, o[0]); o[1] = fmaf(w, u4.y, o[1]); o[2] = fmaf(w, u4.z, o[2]); o[3] = fmaf(w, u4.w, o[3]);
        }
        if (t < count) {
            float* dst = out + ((size_t)(first + t0 + t) * heads + head) * dv + col0 + j0;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (j0 + j < cols) dst[j] = o[j];
        }
        // S0 <- c_C S0 + sum_i (c_C / c_i) k_i u_i^T, four columns of rows t, t + 64, ...
        const float last = lg[CHUNK - 1], cC = expf(last);
        for (int r = t; r < dk; r += CHUNK) {
            float4 s4 = *reinterpret_cast<const float4*>(S0 + r * COLS + j0);
            s4.x *= cC; s4.y *= cC; s4.z *= cC; s4.w *= cC;
#pragma unroll 4
            for (int i = 0; i < count; ++i) {
                const float w = wl[i] * Ks[i * ld + r];
                const float4 u4 = *reinterpret_cast<const float4*>(Bs + i * COLS + j0);
                s4.x = fmaf(w, u4.x, s4.x); s4.y = fmaf(w, u4.y, s4.y); s4.z = fmaf(w, u4.z, s4.z); s4.w = fmaf(w, u4.w, s4.w);
            }
            *reinterpret_cast<float4*>(S0 + r * COLS + j0) = s4;
        }
    }
    __syncthreads();
    for (int i = tid; i < dk * COLS; i += THREADS) {
        const int r = i / COLS, j = i - r * COLS;
        if (j < cols) S[(size_t)r * dv + col0 + j] = S0[i];
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
                                      int dk, int dv, int n_req, int lanes_per_column, int below, void* stream) {
    // `below` > 0: only requests that bring fewer tokens than that (the others run through cisr_delta_chunks)
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
                             qkv, beta, decay, state, state_stride, req_slot, q_start, q_len, out, heads, kvh, dk, dv, below); \
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

CISR_EXPORT int cisr_delta_chunk_tokens() { return CHUNK; }
CISR_EXPORT long long cisr_delta_chunk_table_floats() { return 2 * CHUNK * CHUNK + CHUNK; }

// The recurrence for the requests of the step that bring at least `least` tokens, chunk by chunk.  chunk_req / chunk_t0:
// per chunk its request and first token inside the portion; req_chunk0: per request the index of its first chunk (requests
// below `least` have none); tables: float scratch [n_chunks][heads][cisr_delta_chunk_table_floats()].
CISR_EXPORT int cisr_delta_chunks(const float* qkv, const float* beta, const float* decay, const int* chunk_req, const int* chunk_t0,
                                  int n_chunks, const int* req_chunk0, float* tables, float* state, long long state_stride,
                                  const int* req_slot, const int* q_start, const int* q_len, float* out, int heads, int kvh, int dk,
                                  int dv, int n_req, int least, void* stream) {
    if (n_chunks <= 0 || n_req <= 0) return 0;
    if (dk <= 0 || dk > 256 || dv <= 0 || heads % kvh || least < 1) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem_tables = sizeof(float) * ((size_t)2 * CHUNK * (dk + 1) + 4 * CHUNK * (CHUNK + 1) + 2 * CHUNK);
    const size_t smem_walk = sizeof(float) * ((size_t)2 * CHUNK * chunk_row_stride(dk) + 2 * CHUNK * (CHUNK + 4) + (size_t)dk * 16 +
                                              2 * CHUNK * 16 + 3 * CHUNK);        // sized for 16 columns, also where a CTA takes 8
    if (smem_walk > 220 * 1024) return -3;
    static size_t configured_tables = 48 * 1024, configured_walk = 48 * 1024;
    if (smem_tables > configured_tables) {
        cudaError_t e = cudaFuncSetAttribute(delta_chunk_tables_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_tables);
        if (e != cudaSuccess) return (int)e;
        configured_tables = smem_tables;
    }
    if (smem_walk > configured_walk) {
        cudaError_t e = cudaFuncSetAttribute(delta_chunk_walk_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_walk);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(delta_chunk_walk_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_walk);
        if (e != cudaSuccess) return (int)e;
        configured_walk = smem_walk;
    }
    static int sms = 0;
    if (!sms) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 148;
    }
    const int per_cta = (long long)n_chunks * heads >= 4ll * sms ? heads / kvh : 1;
    int status = launch_kernel(delta_chunk_tables_kernel, dim3(n_chunks, heads / per_cta), dim3(CHUNK_THREADS), smem_tables, s, g_pdl, qkv, beta,
                               decay, chunk_req, chunk_t0, q_start, q_len, tables, heads, kvh, dk, dv, per_cta);
    if (status) return status;
    // 16 value columns per CTA, or 8 where that would leave more than half of the SMs without a CTA (measured: with 128
    // CTAs of 16 columns on 148 SMs, splitting them made the launch slower; with 64 it made it faster)
    if (2ll * n_req * heads * ((dv + 15) / 16) > sms)
        return launch_kernel(delta_chunk_walk_kernel<16>, dim3(n_req, heads, (dv + 15) / 16), dim3(CHUNK * 4), smem_walk, s, g_pdl, qkv, beta,
                             (const float*)tables, req_chunk0, state, state_stride, req_slot, q_start, q_len, out, heads, kvh, dk, dv, least);
    return launch_kernel(delta_chunk_walk_kernel<8>, dim3(n_req, heads, (dv + 7) / 8), dim3(CHUNK * 2), smem_walk, s, g_pdl, qkv, beta,
                         (const float*)tables, req_chunk0, state, state_stride, req_slot, q_start, q_len, out, heads, kvh, dk, dv, least);
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
