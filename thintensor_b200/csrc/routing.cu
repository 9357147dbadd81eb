// Routing of a mixture of experts.
//
// tt_route_topk: one warp per token.  Scores are the softmax of the router's logits over all experts (float32).
// Experts form `groups` equal groups of neighbours; a group's score is its largest expert score, and only experts of
// the `keep` groups with the largest scores can be chosen.  Of those the `top` largest are chosen (ties: the lower
// index), and their weights are their scores divided by the sum of the chosen scores (+ 1e-20).  The kernel writes
// the chosen experts and weights ([tokens][top]) and the same as a dense table ([tokens][experts], zero where an
// expert is not chosen).
//
// tt_route_rows: the same with the router's product in front, from the token's row and the router's matrix.
//
// tt_scale_expert_columns: act[t][e * width + j] *= gates[t][e] for the first experts * width columns of act (the
// columns behind them, a shared expert's, stay as they are).
#include "common.cuh"

constexpr int ROUTE_MAX_EXPERTS = 512;      // a lane holds ROUTE_MAX_EXPERTS / 32 scores
constexpr int ROUTE_WARPS = 4;

// the largest value among the lanes' candidates and the lowest index that has it
__device__ __forceinline__ void route_argmax(float& value, int& index) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, value, o);
        const int i = __shfl_xor_sync(0xffffffffu, index, o);
        if (v > value || (v == value && i < index)) { value = v; index = i; }
    }
}

// One warp routes token t from its logits (`splits` partial sums `split_stride` apart); group_best: 32 floats of the warp's own.
__device__ __forceinline__ void route_token(const float* __restrict__ logits, int splits, size_t split_stride, int t, int experts,
                                            int top, int groups, int keep, float* __restrict__ gates, int* __restrict__ chosen,
                                            float* __restrict__ weights, float* group_best_row) {
    const int lane = threadIdx.x & 31;
    constexpr int PER = ROUTE_MAX_EXPERTS / 32;
    float s[PER];                                               // expert lane + 32 * i
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        s[i] = -INFINITY;
        if (e < experts) {
            float z = 0.0f;
            for (int k = 0; k < splits; ++k) z += logits[(size_t)k * split_stride + e];
            s[i] = z;
            m = fmaxf(m, z);
        }
    }
    m = tt_warp_max(m);
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        if (e < experts) { s[i] = expf(s[i] - m); total += s[i]; } else s[i] = -1.0f;
    }
    total = tt_warp_sum(total);
    const float inv = 1.0f / total;
#pragma unroll
    for (int i = 0; i < PER; ++i)
        if (s[i] >= 0.0f) s[i] *= inv;

    // groups: a bit per group that stays (groups <= 32)
    const int size = experts / groups;
    unsigned kept = 0xffffffffu;
    if (groups > 1 && keep < groups) {
        for (int g = 0; g < groups; ++g) {
            float best = -1.0f;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int e = lane + 32 * i;
                if (e < experts && e / size == g) best = fmaxf(best, s[i]);
            }
            best = tt_warp_max(best);
            if (lane == 0) group_best_row[g] = best;
        }
        __syncwarp();
        kept = 0u;
        for (int round = 0; round < keep; ++round) {
            float v = (lane < groups && !((kept >> lane) & 1u)) ? group_best_row[lane] : -2.0f;
            int g = lane;
            route_argmax(v, g);
            kept |= 1u << g;
        }
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        if (e < experts) gates[(size_t)t * experts + e] = 0.0f;
        if (e < experts && !((kept >> (e / size)) & 1u)) s[i] = -1.0f;
    }
    __syncwarp();

    float sum = 0.0f;
    int mine = -1;                                              // lane r keeps the r-th choice (top <= 32)
    float mine_score = 0.0f;
    for (int round = 0; round < top; ++round) {
        float v = -1.0f;
        int e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (s[i] > v) { v = s[i]; e = lane + 32 * i; }      // a lane's experts rise with i: the first largest is the lowest
        route_argmax(v, e);
        if (v < 0.0f) break;                                    // fewer allowed experts than top
        sum += v;
        if (lane == round) { mine = e; mine_score = v; }
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (lane + 32 * i == e) s[i] = -1.0f;
    }
    const float scale = 1.0f / (sum + 1e-20f);
    if (lane < top) {
        chosen[(size_t)t * top + lane] = mine;
        weights[(size_t)t * top + lane] = mine >= 0 ? mine_score * scale : 0.0f;
        if (mine >= 0) gates[(size_t)t * experts + mine] = mine_score * scale;
    }
}

__global__ void route_topk_kernel(const float* __restrict__ logits, int splits, size_t split_stride, int n_tokens, int experts,
                                  int top, int groups, int keep, float* __restrict__ gates, int* __restrict__ chosen,
                                  float* __restrict__ weights) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    __shared__ float group_best[ROUTE_WARPS][32];
    const int warp = threadIdx.x >> 5;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= n_tokens) return;
    route_token(logits + (size_t)t * experts, splits, split_stride, t, experts, top, groups, keep, gates, chosen, weights, group_best[warp]);
}

// The router's product and the routing in one kernel, one block per token: the token's row goes to shared memory as
// float32, every warp takes experts in turn (lanes across the row, float32 sums), and the first warp then routes the token
// from the logits in shared memory.
template <typename TX, typename TW>
__global__ void route_rows_kernel(const TX* __restrict__ x, const TW* __restrict__ w, int hidden, int n_tokens, int experts, int top,
                                  int groups, int keep, float* __restrict__ gates, int* __restrict__ chosen,
                                  float* __restrict__ weights) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float route_shared[];                     // hidden, then experts, then 32
    float* logits = route_shared + hidden;
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) route_shared[j] = tt_to_float(x[(size_t)t * hidden + j]);
    __syncthreads();
    for (int e = warp; e < experts; e += warps) {
        const TW* row = w + (size_t)e * hidden;
        float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        int j = lane;
        for (; j + 96 < hidden; j += 128) {                     // four loads in flight, four sums
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = tt_to_float(row[j + 32 * i]);
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = fmaf(v[i], route_shared[j + 32 * i], a[i]);
        }
        for (; j < hidden; j += 32) a[0] = fmaf(tt_to_float(row[j]), route_shared[j], a[0]);
        const float z = tt_warp_sum((a[0] + a[1]) + (a[2] + a[3]));
        if (lane == 0) logits[e] = z;
    }
    __syncthreads();
    if (warp == 0) route_token(logits, 1, 0, t, experts, top, groups, keep, gates, chosen, weights, logits + experts);
}

template <typename T>
__global__ void scale_expert_columns_kernel(T* __restrict__ act, int row_stride, int width, int experts,
                                            const float* __restrict__ gates, long long total) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int per_row = experts * width;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row);
    const float g = gates[t * experts + c / width];
    T* p = act + t * row_stride + c;
    *p = tt_from_float<T>(tt_to_float(*p) * g);
}

extern "C" int tt_route_topk(const float* logits, int splits, long long split_stride, int n_tokens, int experts, int top, int groups,
                             int keep, float* gates, int* chosen, float* weights, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (experts <= 0 || experts > ROUTE_MAX_EXPERTS || top < 1 || top > 32 || top > experts || groups < 1 || groups > 32 ||
        experts % groups || keep < 1 || keep > groups)
        return (int)cudaErrorInvalidValue;
    tt_launch_pdl(route_topk_kernel, dim3((n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), 0, stream, logits, splits,
                  (size_t)split_stride, n_tokens, experts, top, groups, keep, gates, chosen, weights);
    TT_LAUNCH_CHECK();
}

// the same, 16 bytes a thread (width and row_stride are multiples of N numbers)
template <typename T, int N>
__global__ void scale_expert_columns_vec_kernel(T* __restrict__ act, int row_stride, int width, int experts,
                                                const float* __restrict__ gates, long long total) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * N;
    if (i >= total) return;
    const int per_row = experts * width;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row);
    const float g = gates[t * experts + c / width];
    uint4* p = reinterpret_cast<uint4*>(act + t * row_stride + c);
    uint4 raw = *p;
    T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int e = 0; e < N; ++e) v[e] = tt_from_float<T>(tt_to_float(v[e]) * g);
    *p = raw;
}

extern "C" int tt_route_rows(const void* x, int x_dtype, const void* w, int w_dtype, int hidden, int n_tokens, int experts, int top,
                             int groups, int keep, float* gates, int* chosen, float* weights, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (experts <= 0 || experts > ROUTE_MAX_EXPERTS || top < 1 || top > 32 || top > experts || groups < 1 || groups > 32 ||
        experts % groups || keep < 1 || keep > groups)
        return (int)cudaErrorInvalidValue;
    const size_t shared = (size_t)(hidden + experts + 32) * sizeof(float);
    if (shared > 48 * 1024) return (int)cudaErrorInvalidValue;
#define TT_ROUTE(TX, TW) tt_launch_pdl(route_rows_kernel<TX, TW>, dim3(n_tokens), dim3(n_tokens <= 256 ? 512 : 128), shared, stream, (const TX*)x, (const TW*)w, hidden, n_tokens, experts, top, groups, keep, gates, chosen, weights)
    if (x_dtype == TT_F32 && w_dtype == TT_F32) TT_ROUTE(float, float);
    else if (x_dtype == TT_F32) TT_ROUTE(float, __nv_bfloat16);
    else if (w_dtype == TT_F32) TT_ROUTE(__nv_bfloat16, float);
    else TT_ROUTE(__nv_bfloat16, __nv_bfloat16);
#undef TT_ROUTE
    TT_LAUNCH_CHECK();
}

extern "C" int tt_scale_expert_columns(void* act, int dtype, int n_tokens, int row_stride, int width, int experts, const float* gates,
                                       cudaStream_t stream) {
    const long long total = (long long)n_tokens * experts * width;
    if (total <= 0) return 0;
    const int threads = 256;
    const int n = dtype == TT_F32 ? 4 : 8;
    if (width % n == 0 && row_stride % n == 0 && ((uintptr_t)act & 15) == 0) {
        const long long blocks = (total / n + threads - 1) / threads;
        if (blocks > 2147483647LL) return (int)cudaErrorInvalidValue;
        if (dtype == TT_F32)
            tt_launch_pdl(scale_expert_columns_vec_kernel<float, 4>, dim3((unsigned)blocks), dim3(threads), 0, stream, (float*)act, row_stride, width, experts, gates, total);
        else
            tt_launch_pdl(scale_expert_columns_vec_kernel<__nv_bfloat16, 8>, dim3((unsigned)blocks), dim3(threads), 0, stream, (__nv_bfloat16*)act, row_stride, width, experts, gates, total);
        TT_LAUNCH_CHECK();
    }
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 2147483647LL) return (int)cudaErrorInvalidValue;
    if (dtype == TT_F32)
        tt_launch_pdl(scale_expert_columns_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, (float*)act, row_stride, width, experts, gates, total);
    else
        tt_launch_pdl(scale_expert_columns_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream, (__nv_bfloat16*)act, row_stride, width, experts, gates, total);
    TT_LAUNCH_CHECK();
}
