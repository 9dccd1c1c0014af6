// From the stacked q | k | v projection of a step to the operands of the paged attention kernels, one CTA per token:
// biases, a norm over a whole projection, rotation of part of each head, heads padded to the width the attention
// kernels are built for, keys and values written into their cache pages.
//
//   row   = proj[t] + bias                                   (bias null: none)
//   qn    = q_norm ? q / sqrt(mean(q^2) + eps) * q_norm : q  (the mean runs over ALL query heads of the token at once)
//   kn    = k_norm ? k / sqrt(mean(k^2) + eps) * k_norm : k
//   q_out[t][h] = [rotate(qn_h) | 0]                          (key_dim wide, padded with zeros to D)
//   k_cache[page][g][off] = [rotate(kn_g) | 0]
//   v_cache[page][g][off] = [v_g | 0]  with v from its own columns, or (v_col < 0) the key as projected: with its bias,
//                                      before norm and rotation; value_dim = key_dim then
//
// The first 2 * rot_half coordinates of a head turn; pairs are (i, i + rot_half) or, interleaved, (2i, 2i + 1).
// The tables hold cos and sin per (token, pair), already multiplied by whatever factor the encoding wants.
// Float arithmetic; one rounding where q_out and the cache have a narrower type.
#include "common.cuh"

static bool g_pdl = false;
CISR_EXPORT void cisr_attention_rows_set_pdl(int on) { g_pdl = on != 0; }

namespace {
__device__ __forceinline__ float turned(const float* head, const float* w, float inv, int d, int rot_half, int interleaved,
                                        const float* cs, const float* sn) {
    // value d of a head after the optional norm (common factor inv, per-coordinate weight w) and the rotation
    float v = head[d] * inv * (w ? w[d] : 1.f);
    if (d < 2 * rot_half) {
        int f, other; bool first;
        if (interleaved) { f = d >> 1; first = !(d & 1); other = first ? d + 1 : d - 1; }
        else { first = d < rot_half; f = first ? d : d - rot_half; other = first ? d + rot_half : d - rot_half; }
        const float o = head[other] * inv * (w ? w[other] : 1.f);
        v = first ? v * cs[f] - o * sn[f] : v * cs[f] + o * sn[f];
    }
    return v;
}

// Coordinates d and d + 1 (d even) of a head after norm and rotation.  Neighbouring pairs turn together, so one pair of
// table entries serves both; the other pairing takes each coordinate's partner from across the head.
__device__ __forceinline__ float2 turned_pair(const float* head, const float* w, float inv, int d, int width, int rot_half,
                                              int interleaved, const float* cs, const float* sn) {
    if (d + 1 >= width || !interleaved || d >= 2 * rot_half)
        return make_float2(d < width ? turned(head, w, inv, d, rot_half, interleaved, cs, sn) : 0.f,
                           d + 1 < width ? turned(head, w, inv, d + 1, rot_half, interleaved, cs, sn) : 0.f);
    const float a = head[d] * inv * (w ? w[d] : 1.f), b = head[d + 1] * inv * (w ? w[d + 1] : 1.f);
    const float c = cs[d >> 1], s = sn[d >> 1];
    return make_float2(a * c - b * s, b * c + a * s);
}
__device__ __forceinline__ void store_pair(float* dst, float2 v) { *reinterpret_cast<float2*>(dst) = v; }
__device__ __forceinline__ void store_pair(__nv_bfloat16* dst, float2 v) { *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v.x, v.y); }

template <typename QT, typename CT>
__global__ void __launch_bounds__(1024)
attention_rows_kernel(const float* __restrict__ proj, int row_stride, int k_col, int v_col, const float* __restrict__ bias,
                      const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_half, int interleaved,
                      QT* __restrict__ q_out, CT* __restrict__ k_cache, CT* __restrict__ v_cache,
                      const int* __restrict__ token_req, const int* __restrict__ positions, const int* __restrict__ req_slot,
                      const int* __restrict__ block_table, int table_width, int page_size, int hq, int hkv, int key_dim,
                      int value_dim, int D, int n_cols) {
    extern __shared__ float row[];            // n_cols floats: the token's projection with its bias
    __shared__ float scratch[32];
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int slot = req_slot[token_req[t]];
    pdl_wait();
    const float* src = proj + (size_t)t * row_stride;
    for (int i = threadIdx.x; i < n_cols; i += blockDim.x) row[i] = src[i] + (bias ? bias[i] : 0.f);
    __syncthreads();
    const int nq = hq * key_dim, nk = hkv * key_dim;
    float inv_q = 1.f, inv_k = 1.f;
    if (q_norm) {
        float sq = 0.f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) sq += row[i] * row[i];
        inv_q = 1.f / sqrtf(block_sum(sq, scratch) / (float)nq + eps);
    }
    if (k_norm) {
        float sq = 0.f;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) sq += row[k_col + i] * row[k_col + i];
        inv_k = 1.f / sqrtf(block_sum(sq, scratch) / (float)nk + eps);
    }
    const float* cs = cos_t ? cos_t + (size_t)t * rot_half : nullptr;
    const float* sn = sin_t ? sin_t + (size_t)t * rot_half : nullptr;
    // a warp per head, a lane per pair of neighbouring coordinates (D is even: pairs never straddle heads)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    for (int h = warp; h < hq; h += n_warps)
        for (int d = 2 * lane; d < D; d += 64)
            store_pair(q_out + ((size_t)t * hq + h) * D + d,
                       turned_pair(row + h * key_dim, q_norm ? q_norm + h * key_dim : nullptr, inv_q, d, key_dim, rot_half, interleaved, cs, sn));
    if (!k_cache) return;
    const int page = block_table[(size_t)slot * table_width + pos / page_size];
    if (page < 0) return;                     // the host reserves a page before every write; never follow a missing entry
    const int off = pos % page_size;
    for (int g = warp; g < hkv; g += n_warps)
        for (int d = 2 * lane; d < D; d += 64) {
            const float* vs = v_col >= 0 ? row + v_col + g * value_dim : row + k_col + g * key_dim;
            const size_t dst = (((size_t)page * hkv + g) * page_size + off) * D + d;
            store_pair(k_cache + dst, turned_pair(row + k_col + g * key_dim, k_norm ? k_norm + g * key_dim : nullptr, inv_k, d, key_dim,
                                                  rot_half, interleaved, cs, sn));
            store_pair(v_cache + dst, make_float2(d < value_dim ? vs[d] : 0.f, d + 1 < value_dim ? vs[d + 1] : 0.f));
        }
}

// out[t][c] += bias[c]
__global__ void bias_add_kernel(float* __restrict__ out, const float* __restrict__ bias, int cols, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] += bias[i % cols];
}
}  // namespace

CISR_EXPORT int cisr_attention_rows(const float* proj, int row_stride, int k_col, int v_col, const float* bias, const float* q_norm,
                                    const float* k_norm, float eps, const float* cos_t, const float* sin_t, int rot_half,
                                    int interleaved, void* q_out, int q_dtype, void* k_cache, void* v_cache, int cache_dtype,
                                    const int* token_req, const int* positions, const int* req_slot, const int* block_table,
                                    int table_width, int page_size, int hq, int hkv, int key_dim, int value_dim, int D, int tokens,
                                    void* stream) {
    if (tokens <= 0) return 0;
    if (2 * rot_half > key_dim || rot_half < 0 || key_dim > D || value_dim > D || hq <= 0 || hkv <= 0) return -2;
    if (v_col < 0 && value_dim != key_dim) return -2;
    if (rot_half && (!cos_t || !sin_t)) return -2;
    const int n_cols = v_col >= 0 ? v_col + hkv * value_dim : k_col + hkv * key_dim;
    if (n_cols > row_stride) return -2;
    const size_t smem = sizeof(float) * (size_t)n_cols;
    if (smem > 200 * 1024) return -3;
    cudaStream_t s = (cudaStream_t)stream;
#define CISR_ROWS(QT, CT)                                                                                                 \
    do {                                                                                                                  \
        static size_t configured = 48 * 1024;                                                                             \
        if (smem > configured) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(attention_rows_kernel<QT, CT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                          \
            configured = smem;                                                                                            \
        }                                                                                                                 \
        /* few tokens (a decode step): a token's row on four times the threads */                                        \
        const int threads = (tokens <= 64 && n_cols >= 1024) ? 1024 : 256;                                                \
        return launch_kernel(attention_rows_kernel<QT, CT>, dim3(tokens), dim3(threads), smem, s, g_pdl, proj, row_stride, k_col, v_col, bias, \
                             q_norm, k_norm, eps, cos_t, sin_t, rot_half, interleaved, (QT*)q_out, (CT*)k_cache, (CT*)v_cache,   \
                             token_req, positions, req_slot, block_table, table_width, page_size, hq, hkv, key_dim, value_dim, D, n_cols); \
    } while (0)
    if (q_dtype == CISR_BF16 && cache_dtype == CISR_BF16) CISR_ROWS(__nv_bfloat16, __nv_bfloat16);
    if (q_dtype == CISR_F32 && cache_dtype == CISR_F32) CISR_ROWS(float, float);
    return -2;
#undef CISR_ROWS
}

CISR_EXPORT int cisr_bias_add(float* out, const float* bias, int rows, int cols, void* stream) {
    const size_t total = (size_t)rows * cols;
    if (!total) return 0;
    bias_add_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(out, bias, cols, total);
    return launch_status();
}
