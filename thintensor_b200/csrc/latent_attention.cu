// Softmax attention over a compressed latent: the cache holds, per token, ONE row of `rank` latent numbers
// followed by `rot` rotated key numbers that all heads share ([block][1][TT_BLOCK_TOKENS][rank + rot], no value
// pool).  A head's keys and values are linear maps of the latent (k_h = Wk_h c, v_h = Wv_h c), so neither is ever
// formed: with a_h = Wk_h^T q_h the score is (a_h . c + q_rot_h . k_rot) * scale, and the head's output is
// Wv_h (sum_j p_j c_j).  Scores, softmax weights, norms, positions and angles are float32 in both dtypes.
//
// tt_latent_prepare: one block per token.  Sums the k-slices of the down projection [q latent | kv latent | k_rot],
// divides the two latents by their root mean square (times their weights), writes the query latent for the
// up projection, rotates k_rot by the token's position and appends [c | k_rot] to the token's cache row.
//
// tt_latent_attention: one warp per (token, head).  Prologue: sums the slices of the head's query, rotates its
// rotated part, forms a_h.  Main loop: a lane per key of a tile of 32 (16-byte loads along the row), online softmax,
// the weighted latents accumulated with lanes across the latent's numbers.  Epilogue: Wv_h times the normalised sum.
// Keys can be cut into slices (decoding long contexts): a slice leaves (sum, maximum, denominator) in scratch memory
// and tt_latent_merge combines the slices in order and applies Wv_h.
#include "attention_kernels.cuh"

constexpr int LAT_WARPS = 4;
constexpr int LAT_MAX_RANK = 512;       // numbers of the latent (a lane accumulates LAT_MAX_RANK / 32 of them)
constexpr int LAT_MAX_ROW = 1024;       // rank + rot
constexpr int LAT_MAX_DIM = 256;        // unrotated numbers of a head's query

template <typename TOut, typename TC>
__global__ void latent_prepare_kernel(const float* __restrict__ down, int splits, size_t split_stride, int q_rank, int rank, int rot,
                                      const float* __restrict__ q_weight, const float* __restrict__ kv_weight, float eps,
                                      const float* __restrict__ inv_freq, int rotary_dim, TOut* __restrict__ q_latent,
                                      TC* __restrict__ pool, const int* __restrict__ table, int table_width, int pool_blocks,
                                      const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                                      unsigned* status) {
    tt_pdl_launch_dependents();
    const int t = blockIdx.x;
    const int b = tt_find_sequence(cu, sequences, t);           // the step's integers are written by no kernel of the step
    const int pos = len_before[b] + (t - cu[b]);
    tt_pdl_wait();
    extern __shared__ float lat_row[];                          // q_rank + rank + rot numbers, then 32 for the reductions
    const int cols = q_rank + rank + rot;
    float* reduce = lat_row + cols;
    const float* src = down + (size_t)t * cols;
    float sq_q = 0.0f, sq_c = 0.0f;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) {
        float x = 0.0f;
        for (int s = 0; s < splits; ++s) x += src[(size_t)s * split_stride + j];
        lat_row[j] = x;
        if (j < q_rank) sq_q = fmaf(x, x, sq_q);
        else if (j < q_rank + rank) sq_c = fmaf(x, x, sq_c);
    }
    const float r_q = rsqrtf(tt_block_sum(sq_q, reduce) / (float)q_rank + eps);
    const float r_c = rsqrtf(tt_block_sum(sq_c, reduce) / (float)rank + eps);
    for (int j = threadIdx.x; j < q_rank; j += blockDim.x)
        q_latent[(size_t)t * q_rank + j] = tt_from_float<TOut>(lat_row[j] * r_q * __ldg(q_weight + j));
    if (!pool) return;
    const long long off = tt_cache_offset(table + (size_t)b * table_width, pos, 0, 1, rank + rot, pool_blocks, status);
    if (off < 0) return;
    TC* row = pool + off;
    const float* c = lat_row + q_rank;
    for (int j = threadIdx.x; j < rank; j += blockDim.x) row[j] = tt_from_float<TC>(c[j] * r_c * __ldg(kv_weight + j));
    const float* kr = c + rank;
    const int half = rotary_dim >> 1;
    for (int j = threadIdx.x; j < rot; j += blockDim.x) {
        float v = kr[j];
        if (j < rotary_dim) {
            const int i = j < half ? j : j - half;
            float sn, cs;
            sincosf((float)pos * __ldg(inv_freq + i), &sn, &cs);
            v = j < half ? kr[j] * cs - kr[j + half] * sn : kr[j] * cs + kr[j - half] * sn;
        }
        row[rank + j] = tt_from_float<TC>(v);
    }
}

template <typename T> __device__ __forceinline__ float lat_weight(const T* p) { return tt_to_float(*p); }

// window <= 0: all keys 0..pos.  window > 0: keys pos - window + 1 .. pos.
template <typename TOut, typename TC, typename TW>
__global__ void latent_attention_kernel(const float* __restrict__ q, int q_splits, size_t q_stride, const TW* __restrict__ w_key,
                                        const TW* __restrict__ w_value, const TC* __restrict__ pool, const int* __restrict__ table,
                                        int table_width, int pool_blocks, const int* __restrict__ cu,
                                        const int* __restrict__ len_before, int sequences, int n_tokens, int heads, int dim, int rot,
                                        int vdim, int rank, const float* __restrict__ inv_freq, int rotary_dim, float scale,
                                        int window, int splits, TOut* __restrict__ out, float* __restrict__ part_acc,
                                        float* __restrict__ part_ml, unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float lat_shared[];                       // per warp: rank + rot (the absorbed query), then dim
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * LAT_WARPS + warp;   // (token, head)
    if (item >= (long long)n_tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
    const int split = blockIdx.y;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    const int* table_row = table + (size_t)b * table_width;
    const int row_len = rank + rot;
    float* qa = lat_shared + (size_t)warp * (row_len + dim);
    float* qp = qa + row_len;

    // the head's query: dim unrotated numbers, then rot numbers of which the first rotary_dim are rotated
    const float* qsrc = q + ((size_t)t * heads + h) * (dim + rot);
    for (int d = lane; d < dim + rot; d += 32) {
        float x = 0.0f;
        for (int s = 0; s < q_splits; ++s) x += qsrc[(size_t)s * q_stride + d];
        if (d < dim) qp[d] = x; else qa[rank + d - dim] = x;
    }
    __syncwarp();
    {
        const int half = rotary_dim >> 1;
        float* qr = qa + rank;
        for (int i = lane; i < half; i += 32) {
            float sn, cs;
            sincosf((float)pos * __ldg(inv_freq + i), &sn, &cs);
            const float u = qr[i], v = qr[i + half];
            qr[i] = (u * cs - v * sn) * scale;
            qr[i + half] = (v * cs + u * sn) * scale;
        }
        for (int i = rotary_dim + lane; i < rot; i += 32) qr[i] *= scale;
    }
    // a = Wk_h^T q (rank numbers): lanes across the latent, so that a row of Wk_h is read side by side
    float acc[LAT_MAX_RANK / 32];
#pragma unroll
    for (int i = 0; i < LAT_MAX_RANK / 32; ++i) acc[i] = 0.0f;
    for (int d = 0; d < dim; ++d) {
        const float qd = qp[d];
        const TW* wrow = w_key + ((size_t)h * dim + d) * rank;
#pragma unroll
        for (int i = 0; i < LAT_MAX_RANK / 32; ++i) {
            const int r = lane + 32 * i;
            if (r < rank) acc[i] = fmaf(lat_weight(wrow + r), qd, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < LAT_MAX_RANK / 32; ++i) {
        const int r = lane + 32 * i;
        if (r < rank) qa[r] = acc[i] * scale;
        acc[i] = 0.0f;
    }
    __syncwarp();

    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_keys = pos - first + 1;
    int per = (n_keys + splits - 1) / splits;
    per = (per + 31) & ~31;
    const int begin = first + split * per;
    const int end = min(begin + per, pos + 1);

    float m_run = -INFINITY, l_run = 0.0f;
    for (int base = begin; base < end; base += 32) {
        const int key = base + lane;
        long long off = -1;
        float score = -INFINITY;
        if (key < end) {
            off = tt_cache_offset(table_row, key, 0, 1, row_len, pool_blocks, status);
            if (off >= 0) score = dot16<TC>(pool + off, qa, row_len);
        }
        const float m_tile = tt_warp_max(score);
        if (m_tile == -INFINITY) continue;
        const float m_new = fmaxf(m_run, m_tile);
        const float corr = expf(m_run - m_new);
        const float p = (score == -INFINITY) ? 0.0f : expf(score - m_new);
        l_run = l_run * corr + tt_warp_sum(p);
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < LAT_MAX_RANK / 32; ++i) acc[i] *= corr;
        const int count = min(32, end - base);
        for (int j = 0; j < count; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long oj = __shfl_sync(0xffffffffu, off, j);
            if (oj < 0) continue;
            const TC* crow = pool + oj;                         // the key's latent is also its value
#pragma unroll
            for (int i = 0; i < LAT_MAX_RANK / 32; ++i) {
                const int r = lane + 32 * i;
                if (r < rank) acc[i] = fmaf(pj, tt_to_float(crow[r]), acc[i]);
            }
        }
    }

    if (splits > 1) {
        const size_t slot = ((size_t)t * heads + h) * splits + split;
#pragma unroll
        for (int i = 0; i < LAT_MAX_RANK / 32; ++i) {
            const int r = lane + 32 * i;
            if (r < rank) part_acc[slot * rank + r] = acc[i];
        }
        if (lane == 0) {
            part_ml[slot * 2] = m_run;
            part_ml[slot * 2 + 1] = l_run;
        }
        return;
    }
    // the head's output: Wv_h times the normalised sum of latents
    const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < LAT_MAX_RANK / 32; ++i) {
        const int r = lane + 32 * i;
        if (r < rank) qa[r] = acc[i] * inv;
    }
    __syncwarp();
    for (int v0 = 0; v0 < vdim; v0 += 32) {
        const int v = v0 + lane;
        float o = 0.0f;
        if (v < vdim) {
            const TW* wrow = w_value + ((size_t)h * vdim + v) * rank;
            for (int r = 0; r < rank; ++r) o = fmaf(lat_weight(wrow + r), qa[r], o);
            out[((size_t)t * heads + h) * vdim + v] = tt_from_float<TOut>(o);
        }
    }
}

// Combines the key slices of one (token, head) in slice order and applies Wv_h.  One warp per row.
template <typename TOut, typename TW>
__global__ void latent_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int splits, int rank,
                                    int vdim, int heads, long long rows, const TW* __restrict__ w_value, TOut* __restrict__ out) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float lat_shared[];                       // per warp: rank
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * LAT_WARPS + warp;
    if (row >= rows) return;
    const int h = (int)(row % heads);
    float* o_lat = lat_shared + (size_t)warp * rank;
    const float* ml = part_ml + (size_t)row * splits * 2;
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, ml[2 * s]);
    float l = 0.0f;
    float acc[LAT_MAX_RANK / 32];
#pragma unroll
    for (int i = 0; i < LAT_MAX_RANK / 32; ++i) acc[i] = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float ms = ml[2 * s];
        if (ms == -INFINITY) continue;
        const float w = expf(ms - m);
        l += ml[2 * s + 1] * w;
        const float* a = part_acc + ((size_t)row * splits + s) * rank;
#pragma unroll
        for (int i = 0; i < LAT_MAX_RANK / 32; ++i) {
            const int r = lane + 32 * i;
            if (r < rank) acc[i] = fmaf(a[r], w, acc[i]);
        }
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < LAT_MAX_RANK / 32; ++i) {
        const int r = lane + 32 * i;
        if (r < rank) o_lat[r] = acc[i] * inv;
    }
    __syncwarp();
    for (int v0 = 0; v0 < vdim; v0 += 32) {
        const int v = v0 + lane;
        if (v < vdim) {
            float o = 0.0f;
            const TW* wrow = w_value + ((size_t)h * vdim + v) * rank;
            for (int r = 0; r < rank; ++r) o = fmaf(lat_weight(wrow + r), o_lat[r], o);
            out[(size_t)row * vdim + v] = tt_from_float<TOut>(o);
        }
    }
}

extern "C" int tt_latent_prepare(const float* down, int splits, long long split_stride, int q_rank, int rank, int rot,
                                 const float* q_weight, const float* kv_weight, float eps, const float* inv_freq, int rotary_dim,
                                 void* q_latent, int act_dtype, void* pool, int cache_dtype, const int* table, int table_width,
                                 int pool_blocks, const int* cu, const int* len_before, int sequences, int n_tokens, unsigned* status,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rank <= 0 || q_rank <= 0 || rot < 0 || rotary_dim < 0 || rotary_dim > rot || (rotary_dim & 1) || act_dtype != cache_dtype)
        return (int)cudaErrorInvalidValue;
    const int cols = q_rank + rank + rot;
    const size_t shared = (size_t)(cols + 32) * sizeof(float);
    if (shared > 48 * 1024) return (int)cudaErrorInvalidValue;
    const int threads = cols >= 1024 ? 256 : 128;
#define TT_PREP(T) tt_launch_pdl(latent_prepare_kernel<T, T>, dim3(n_tokens), dim3(threads), shared, stream, down, splits, (size_t)split_stride, q_rank, rank, rot, q_weight, kv_weight, eps, inv_freq, rotary_dim, (T*)q_latent, (T*)pool, table, table_width, pool_blocks, cu, len_before, sequences, status)
    if (act_dtype == TT_F32) TT_PREP(float); else TT_PREP(__nv_bfloat16);
#undef TT_PREP
    TT_LAUNCH_CHECK();
}

extern "C" int tt_latent_attention(const float* q, int q_splits, long long q_stride, const void* w_key, const void* w_value,
                                   int weight_dtype, const void* pool, int act_dtype, const int* table, int table_width, int pool_blocks,
                                   const int* cu, const int* len_before, int sequences, int n_tokens, int heads, int dim, int rot,
                                   int vdim, int rank, const float* inv_freq, int rotary_dim, float scale, int window, int splits,
                                   void* out, float* part_acc, float* part_ml, unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rank <= 0 || rank > LAT_MAX_RANK || rank + rot > LAT_MAX_ROW || dim <= 0 || dim > LAT_MAX_DIM || vdim <= 0 || splits < 1 ||
        splits > 65535 || rotary_dim > rot || (rotary_dim & 1) || (splits > 1 && (!part_acc || !part_ml)))
        return (int)cudaErrorInvalidValue;
    const long long rows = (long long)n_tokens * heads;
    const long long blocks = (rows + LAT_WARPS - 1) / LAT_WARPS;
    if (blocks > 2147483647LL) return (int)cudaErrorInvalidValue;
    const size_t shared = (size_t)LAT_WARPS * (rank + rot + dim) * sizeof(float);
    const dim3 grid((unsigned)blocks, splits), block(LAT_WARPS * 32);
#define TT_ATT(TA, TW) tt_launch_pdl(latent_attention_kernel<TA, TA, TW>, grid, block, shared, stream, q, q_splits, (size_t)q_stride, (const TW*)w_key, (const TW*)w_value, (const TA*)pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, dim, rot, vdim, rank, inv_freq, rotary_dim, scale, window, splits, (TA*)out, part_acc, part_ml, status)
#define TT_MERGE(TA, TW) tt_launch_pdl(latent_merge_kernel<TA, TW>, dim3((unsigned)blocks), block, (size_t)LAT_WARPS * rank * sizeof(float), stream, (const float*)part_acc, (const float*)part_ml, splits, rank, vdim, heads, rows, (const TW*)w_value, (TA*)out)
    if (act_dtype == TT_F32 && weight_dtype == TT_F32) { TT_ATT(float, float); if (splits > 1) TT_MERGE(float, float); }
    else if (act_dtype == TT_F32) { TT_ATT(float, __nv_bfloat16); if (splits > 1) TT_MERGE(float, __nv_bfloat16); }
    else if (weight_dtype == TT_F32) { TT_ATT(__nv_bfloat16, float); if (splits > 1) TT_MERGE(__nv_bfloat16, float); }
    else { TT_ATT(__nv_bfloat16, __nv_bfloat16); if (splits > 1) TT_MERGE(__nv_bfloat16, __nv_bfloat16); }
#undef TT_ATT
#undef TT_MERGE
    TT_LAUNCH_CHECK();
}
