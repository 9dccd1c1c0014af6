// Latent attention: the small kernels around its matrix products.
//
// A token's keys and values are kept as one row of the cache: the normed latent c (kv_rank wide) followed by the
// rotated key part that all heads share (rot_dim wide), padded with zeros to the cache's row width.  Queries are
// brought to the same basis (q_h -> [W_uk_h^T q_h,plain | rotated part]) so attention runs over the rows as they are
// stored, with the row's first kv_rank columns as the value; the value projection W_uv_h follows the weighted sum.
//
// Everything here is float arithmetic: unit norms, rotation (tables come in float from float64 angles), the gate's
// sigmoid.  Storage is rounded once, on the way out.
#include "common.cuh"

static bool g_pdl = false;
CISR_EXPORT void cisr_latent_set_pdl(int on) { g_pdl = on != 0; }

// Rotated value of coordinate d (< 2 * rot_half) of a vector whose float coordinates are src[0 .. 2 * rot_half).
__device__ __forceinline__ float rotated(const float* __restrict__ src, int d, int rot_half, int interleaved,
                                         const float* __restrict__ cs, const float* __restrict__ sn) {
    int f, other; bool first;
    if (interleaved) { f = d >> 1; first = !(d & 1); other = first ? d + 1 : d - 1; }
    else { first = d < rot_half; f = first ? d : d - rot_half; other = first ? d + rot_half : d - rot_half; }
    const float c = cs[f], s = sn[f], v = src[d], o = src[other];
    return first ? v * c - o * s : v * c + o * s;
}

// ---------------------------------------------------------------- down projections -> latents and cache row
// proj [T, row_stride] float holds, per token, the query latent at q_col (q_rank wide; q_rank 0: none), the key/value
// latent at c_col (kv_rank wide) and right behind it the shared key part (2 * rot_half wide).
//   cq_out[t]            = unit(proj[q_col ..]) * q_norm_w                      (storage type of the next product)
//   cache row of token t = [unit(proj[c_col ..]) * c_norm_w | rotate(key part) | 0 ...]
// unit(v) = v / sqrt(mean(v^2) + eps).  The row lies in page block_table[slot][pos / P] at offset pos % P of a cache
// laid out [pages, 1, P, row_width].
template <typename CT>
__global__ void latent_rows_kernel(const float* __restrict__ proj, int row_stride, int q_col, int q_rank,
                                   const float* __restrict__ q_norm_w, CT* __restrict__ cq_out, int c_col, int kv_rank,
                                   const float* __restrict__ c_norm_w, float eps, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, int rot_half, int interleaved, CT* __restrict__ cache,
                                   int row_width, const int* __restrict__ token_req, const int* __restrict__ positions,
                                   const int* __restrict__ req_slot, const int* __restrict__ block_table, int table_width,
                                   int page_size) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * row_stride;
    if (q_rank > 0) {
        float sq = 0.f;
        for (int d = threadIdx.x; d < q_rank; d += blockDim.x) { const float v = row[q_col + d]; sq += v * v; }
        const float unit = rsqrtf(block_sum(sq, scratch) / (float)q_rank + eps);
        for (int d = threadIdx.x; d < q_rank; d += blockDim.x)
            cq_out[(size_t)t * q_rank + d] = from_float<CT>(row[q_col + d] * unit * q_norm_w[d]);
    }
    if (!cache) return;
    float sq = 0.f;
    for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) { const float v = row[c_col + d]; sq += v * v; }
    const float unit = rsqrtf(block_sum(sq, scratch) / (float)kv_rank + eps);
    const int pos = positions[t];
    const int page = block_table[(size_t)req_slot[token_req[t]] * table_width + pos / page_size];
    if (page < 0) return;      // the host reserves a page before every write; never follow a missing entry
    CT* dst = cache + ((size_t)page * page_size + pos % page_size) * row_width;
    const float* key = row + c_col + kv_rank;
    const float* cs = cos_t + (size_t)t * rot_half;
    const float* sn = sin_t + (size_t)t * rot_half;
    for (int d = threadIdx.x; d < row_width; d += blockDim.x) {
        float v = 0.f;
        if (d < kv_rank) v = row[c_col + d] * unit * c_norm_w[d];
        else if (d < kv_rank + 2 * rot_half) v = rotated(key, d - kv_rank, rot_half, interleaved, cs, sn);
        dst[d] = from_float<CT>(v);
    }
}

CISR_EXPORT int cisr_latent_rows(const float* proj, int row_stride, int q_col, int q_rank, const float* q_norm_w, void* cq_out,
                                 int c_col, int kv_rank, const float* c_norm_w, float eps, const float* cos_t,
                                 const float* sin_t, int rot_half, int interleaved, void* cache, int row_width, int dtype,
                                 const int* token_req, const int* positions, const int* req_slot, const int* block_table,
                                 int table_width, int page_size, int tokens, void* stream) {
    if (tokens <= 0) return 0;
    if (kv_rank + 2 * rot_half > row_width || rot_half < 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CISR_BF16)
        return launch_kernel(latent_rows_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, s, g_pdl, proj, row_stride, q_col, q_rank,
                             q_norm_w, (__nv_bfloat16*)cq_out, c_col, kv_rank, c_norm_w, eps, cos_t, sin_t, rot_half, interleaved,
                             (__nv_bfloat16*)cache, row_width, token_req, positions, req_slot, block_table, table_width, page_size);
    return launch_kernel(latent_rows_kernel<float>, dim3(tokens), dim3(128), 0, s, g_pdl, proj, row_stride, q_col, q_rank, q_norm_w,
                         (float*)cq_out, c_col, kv_rank, c_norm_w, eps, cos_t, sin_t, rot_half, interleaved, (float*)cache, row_width,
                         token_req, positions, req_slot, block_table, table_width, page_size);
}

// ---------------------------------------------------------------- queries: split and rotate
// q [T, row_stride] float holds heads of [plain | rotated part] (plain_dim + 2 * rot_half wide) from column q_col on.
//   plain_out[t, h, :]                          = the plain part (operand of the product with W_uk_h)
//   q_rows[t, h, kv_rank .. kv_rank + rot)      = the rotated part, turned to the token's position
//   q_rows[t, h, kv_rank + rot .. row_width)    = 0
// q_rows[t, h, 0 .. kv_rank) is written by that product.
template <typename CT>
__global__ void latent_query_kernel(const float* __restrict__ q, int row_stride, int q_col, int heads, int plain_dim,
                                    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_half,
                                    int interleaved, CT* __restrict__ plain_out, CT* __restrict__ q_rows, int kv_rank,
                                    int row_width) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, rot = 2 * rot_half, head_w = plain_dim + rot;
    const float* row = q + (size_t)t * row_stride + q_col;
    const float* cs = cos_t + (size_t)t * rot_half;
    const float* sn = sin_t + (size_t)t * rot_half;
    for (int i = threadIdx.x; i < heads * plain_dim; i += blockDim.x) {
        const int h = i / plain_dim, d = i - h * plain_dim;
        plain_out[(size_t)t * heads * plain_dim + i] = from_float<CT>(row[h * head_w + d]);
    }
    const int tail = row_width - kv_rank;
    for (int i = threadIdx.x; i < heads * tail; i += blockDim.x) {
        const int h = i / tail, d = i - h * tail;
        const float v = d < rot ? rotated(row + h * head_w + plain_dim, d, rot_half, interleaved, cs, sn) : 0.f;
        q_rows[((size_t)t * heads + h) * row_width + kv_rank + d] = from_float<CT>(v);
    }
}

CISR_EXPORT int cisr_latent_query(const float* q, int row_stride, int q_col, int heads, int plain_dim, const float* cos_t,
                                  const float* sin_t, int rot_half, int interleaved, void* plain_out, void* q_rows,
                                  int kv_rank, int row_width, int dtype, int tokens, void* stream) {
    if (tokens <= 0) return 0;
    if (kv_rank + 2 * rot_half > row_width) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CISR_BF16)
        return launch_kernel(latent_query_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, s, g_pdl, q, row_stride, q_col, heads,
                             plain_dim, cos_t, sin_t, rot_half, interleaved, (__nv_bfloat16*)plain_out, (__nv_bfloat16*)q_rows,
                             kv_rank, row_width);
    return launch_kernel(latent_query_kernel<float>, dim3(tokens), dim3(256), 0, s, g_pdl, q, row_stride, q_col, heads, plain_dim,
                         cos_t, sin_t, rot_half, interleaved, (float*)plain_out, (float*)q_rows, kv_rank, row_width);
}

// ---------------------------------------------------------------- output gate
// out[t, i] = values[t, i] * sigmoid(gate[t, gate_col + i]) (gate null: out = values), rounded to the storage type of
// the output projection's operand.
template <typename CT>
__global__ void latent_gate_kernel(const float* __restrict__ values, const float* __restrict__ gate, int gate_stride,
                                   int gate_col, CT* __restrict__ out, int width, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float v = values[i];
    if (gate) {
        const size_t t = i / width;
        const float g = gate[t * gate_stride + gate_col + (i - t * width)];
        v *= 1.f / (1.f + expf(-g));
    }
    out[i] = from_float<CT>(v);
}

CISR_EXPORT int cisr_latent_gate(const float* values, const float* gate, int gate_stride, int gate_col, void* out, int dtype,
                                 int tokens, int width, void* stream) {
    const size_t total = (size_t)tokens * width;
    if (!total) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((unsigned)((total + 255) / 256));
    if (dtype == CISR_BF16)
        return launch_kernel(latent_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, g_pdl, values, gate, gate_stride, gate_col,
                             (__nv_bfloat16*)out, width, total);
    return launch_kernel(latent_gate_kernel<float>, grid, dim3(256), 0, s, g_pdl, values, gate, gate_stride, gate_col, (float*)out,
                         width, total);
}

// ---------------------------------------------------------------- few tokens: the per-head products as row kernels
// With a handful of tokens (decode steps) the two products per head are too small for a library call each: a CTA per
// (token, head) reads its head's matrix straight from L2.
//
// latent_absorb: the work of latent_query and of the product with W_kup in one launch.
//   q_rows[t, h, r]              = sum_d round(q[t, h, d]) * W_kup[h][d][r]     r < kv_rank, d < plain_dim
//   q_rows[t, h, kv_rank + ..]   = rotated part, then zeros
// (the plain part is rounded to the storage type first, as the operand of the library product is).
constexpr int ABSORB_SPLIT = 4;       // the sum over a head's plain coordinates is cut into this many parts, each with its loads in flight at once
template <typename CT>
__global__ void latent_absorb_kernel(const float* __restrict__ q, int row_stride, int q_col, int heads, int plain_dim,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_half, int interleaved,
                                     const CT* __restrict__ k_up, CT* __restrict__ q_rows, int kv_rank, int row_width) {
    extern __shared__ float absorb_smem[];      // plain_dim floats, then ABSORB_SPLIT * kv_rank partial sums
    float* plain = absorb_smem;
    float* part = absorb_smem + plain_dim;
    pdl_trigger();
    const int t = blockIdx.x, h = blockIdx.y, rot = 2 * rot_half;
    const CT* w = k_up + (size_t)h * plain_dim * kv_rank;
    pdl_wait();
    const float* row = q + (size_t)t * row_stride + q_col + (size_t)h * (plain_dim + rot);
    for (int d = threadIdx.x; d < plain_dim; d += blockDim.x) plain[d] = to_float(from_float<CT>(row[d]));
    __syncthreads();
    const int per = (plain_dim + ABSORB_SPLIT - 1) / ABSORB_SPLIT;
    for (int i = threadIdx.x; i < ABSORB_SPLIT * kv_rank; i += blockDim.x) {
        const int g = i / kv_rank, r = i - g * kv_rank, d0 = g * per, d1 = min(plain_dim, d0 + per);
        float acc = 0.f;
#pragma unroll 8
        for (int d = d0; d < d1; ++d) acc += plain[d] * to_float(w[(size_t)d * kv_rank + r]);
        part[i] = acc;
    }
    __syncthreads();
    CT* dst = q_rows + ((size_t)t * heads + h) * row_width;
    for (int r = threadIdx.x; r < row_width; r += blockDim.x) {
        float acc = 0.f;
        if (r < kv_rank) {
#pragma unroll
            for (int g = 0; g < ABSORB_SPLIT; ++g) acc += part[g * kv_rank + r];       // the parts in their fixed order
        } else if (r < kv_rank + rot) {
            acc = rotated(row + plain_dim, r - kv_rank, rot_half, interleaved, cos_t + (size_t)t * rot_half, sin_t + (size_t)t * rot_half);
        }
        dst[r] = from_float<CT>(acc);
    }
}

CISR_EXPORT int cisr_latent_absorb(const float* q, int row_stride, int q_col, int heads, int plain_dim, const float* cos_t,
                                   const float* sin_t, int rot_half, int interleaved, const void* k_up, void* q_rows, int kv_rank,
                                   int row_width, int dtype, int tokens, void* stream) {
    if (tokens <= 0) return 0;
    if (kv_rank + 2 * rot_half > row_width) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(tokens, heads);
    const size_t smem = sizeof(float) * ((size_t)plain_dim + (size_t)ABSORB_SPLIT * kv_rank);
    if (smem > 48 * 1024) return -3;
    const int threads = ABSORB_SPLIT * kv_rank >= 512 ? 512 : (ABSORB_SPLIT * kv_rank >= 256 ? 256 : 128);
    if (dtype == CISR_BF16)
        return launch_kernel(latent_absorb_kernel<__nv_bfloat16>, grid, dim3(threads), smem, s, g_pdl, q, row_stride, q_col, heads, plain_dim,
                             cos_t, sin_t, rot_half, interleaved, (const __nv_bfloat16*)k_up, (__nv_bfloat16*)q_rows, kv_rank, row_width);
    return launch_kernel(latent_absorb_kernel<float>, grid, dim3(threads), smem, s, g_pdl, q, row_stride, q_col, heads, plain_dim, cos_t,
                         sin_t, rot_half, interleaved, (const float*)k_up, (float*)q_rows, kv_rank, row_width);
}

// latent_values: the product with W_vup and the output gate in one launch.
//   out[t, h * value_dim + j] = (sum_r mixed[t, h, r] * W_vup[h][j][r]) * sigmoid(gate[t, gate_col + h * value_dim + j])
// mixed [tokens, heads, row_width] is the attention's weighted sum of cache rows (its first kv_rank columns count);
// gate null: no gate.  A warp per output feature, its lanes striding over the latent.
template <typename CT>
__global__ void latent_values_kernel(const CT* __restrict__ mixed, int heads, int row_width, int kv_rank, const CT* __restrict__ v_up,
                                     int value_dim, const float* __restrict__ gate, int gate_stride, int gate_col, CT* __restrict__ out) {
    pdl_trigger();
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int warp = blockIdx.z * n_warps + (threadIdx.x >> 5), all_warps = gridDim.z * n_warps;    // a warp has one feature when the grid is large enough
    const CT* w = v_up + (size_t)h * value_dim * kv_rank;
    pdl_wait();
    const CT* m = mixed + ((size_t)t * heads + h) * row_width;
    for (int j = warp; j < value_dim; j += all_warps) {
        float acc = 0.f;
        for (int r = lane; r < kv_rank; r += 32) acc += to_float(m[r]) * to_float(w[(size_t)j * kv_rank + r]);
        acc = warp_sum(acc);
        if (lane == 0) {
            const int col = h * value_dim + j;
            if (gate) acc *= 1.f / (1.f + expf(-gate[(size_t)t * gate_stride + gate_col + col]));
            out[(size_t)t * heads * value_dim + col] = from_float<CT>(acc);
        }
    }
}

CISR_EXPORT int cisr_latent_values(const void* mixed, int heads, int row_width, int kv_rank, const void* v_up, int value_dim,
                                   const float* gate, int gate_stride, int gate_col, void* out, int dtype, int tokens, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(tokens, heads, (value_dim + 7) / 8);
    if (dtype == CISR_BF16)
        return launch_kernel(latent_values_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, g_pdl, (const __nv_bfloat16*)mixed, heads, row_width,
                             kv_rank, (const __nv_bfloat16*)v_up, value_dim, gate, gate_stride, gate_col, (__nv_bfloat16*)out);
    return launch_kernel(latent_values_kernel<float>, grid, dim3(256), 0, s, g_pdl, (const float*)mixed, heads, row_width, kv_rank,
                         (const float*)v_up, value_dim, gate, gate_stride, gate_col, (float*)out);
}
