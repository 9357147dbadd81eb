// Kernels of the recurrent token mixers: the short causal convolution with its carried inputs, the
// Mamba-2 state-space recurrence (also run with a constant decay and step size one: the linear
// attention S <- g S + k v^T, o = S^T q, whose q, k and v a kernel here prepares), the gated delta-rule
// recurrence, the gated group norm behind them (gate: silu or sigmoid), and the weighted sum of two branches.  Everything here is float32: inputs are the float32 partial
// sums of a projection ([splits][tokens][cols], summed on the way in), states live in float32 and are
// carried per sequence slot, and only the normalised output that feeds the next matrix product is
// narrowed to the activation dtype.
//
// Packed batches: token t belongs to the sequence b with cu[b] <= t < cu[b + 1]; its state lies at
// slots[b].  A recurrence walks a sequence's tokens in order and starts from the slot's state, so a
// prompt cut into steps, a prompt and its decoded tokens, and a sequence inside a batch all run the
// same chain of operations and give the same bits.
//
// A state matrix is owned column by column: the column of value dimension p (all its N state rows)
// belongs to a group of REC_LANES neighbouring lanes, lane l holding rows 4l .. 4l + 3, 4l + 32 .. 4l + 35, ...
// in registers (four neighbouring rows at a time, so that a token's vectors come out of shared memory, and the
// state out of global memory, in 16-byte pieces that the group's lanes read side by side).  Row products with the token's vectors (read from shared memory, where a chunk of tokens
// is staged) are summed inside the group with shuffles.  Columns are independent, so a CTA takes
// REC_COLS of them for one (sequence, head) and the grid is heads x sequences x column tiles.  When that
// grid would fill the GPU more than twice over, a lane group owns four neighbouring columns instead and
// a CTA 64 of them (see the kernels' template parameters).
#include "common.cuh"

constexpr int REC_LANES = 8;        // lanes that share one state column (measured on a B200, 64 heads of 64 x 128: one sequence of 2,048
                                    // tokens 0.79 ms with 8 lanes and 0.86 ms with 16; one token of 64 sequences 70 us and 94 us)
constexpr int REC_COLS = 32;        // state columns of a CTA (REC_COLS * REC_LANES threads)
constexpr int REC_CHUNK = 16;       // tokens staged in shared memory at a time
constexpr int REC_MAX_ROWS = 256;   // largest state size per column (N of Mamba-2, key size of the delta rule)
constexpr int CONV_MAX_TAPS = 8;

// sum of one element over the k-slices of a projection: four loads in flight together, additions in slice order
__device__ __forceinline__ float rec_sum_slices(const float* __restrict__ p, int splits, size_t split_stride) {
    float total = 0.0f;
    int s = 0;
    for (; s + 4 <= splits; s += 4) {
        const float a = __ldg(p + (size_t)s * split_stride), b = __ldg(p + (size_t)(s + 1) * split_stride);
        const float c = __ldg(p + (size_t)(s + 2) * split_stride), d = __ldg(p + (size_t)(s + 3) * split_stride);
        total = (((total + a) + b) + c) + d;
    }
    for (; s < splits; ++s) total += __ldg(p + (size_t)s * split_stride);
    return total;
}

// Asynchronous copies into shared memory: a chunk of tokens is fetched while the chunk before it is worked on.
__device__ __forceinline__ uint32_t rec_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void rec_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(rec_smem(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void rec_copy16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(rec_smem(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void rec_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void rec_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// rows x width floats from src (row stride src_stride) to dst (row stride dst_stride), all threads of the block taking
// part; vec: every row start and the width are multiples of four floats and both bases are 16-byte aligned
__device__ __forceinline__ void rec_stage(float* dst, int dst_stride, const float* src, size_t src_stride, int rows, int width, bool vec) {
    if (vec) {
        const int quads = width >> 2;
        for (int e = threadIdx.x; e < rows * quads; e += blockDim.x) {
            const int k = e / quads, r = (e - k * quads) << 2;
            rec_copy16(dst + k * dst_stride + r, src + (size_t)k * src_stride + r);
        }
    } else {
        for (int e = threadIdx.x; e < rows * width; e += blockDim.x) {
            const int k = e / width, r = e - k * width;
            rec_copy4(dst + k * dst_stride + r, src + (size_t)k * src_stride + r);
        }
    }
}

__device__ __forceinline__ float rec_silu(float x) { return x / (1.0f + expf(-x)); }
// the gate of a normed read-out: 0 silu, 1 sigmoid
__device__ __forceinline__ float rec_gate(float x, int kind) { return kind == 1 ? 1.0f / (1.0f + expf(-x)) : rec_silu(x); }
__device__ __forceinline__ float rec_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// the state row that register i of lane `lane` holds
__device__ __forceinline__ int rec_row(int lane, int i) { return 4 * lane + 4 * REC_LANES * (i >> 2) + (i & 3); }

// a column's registers from / to its N numbers in global memory
template <int K>
__device__ __forceinline__ void rec_load_column(float (&s)[K], const float* __restrict__ S, int lane, int N, bool live) {
#pragma unroll
    for (int j = 0; j < K / 4; ++j) {
        const int r = rec_row(lane, 4 * j);
        if (live && !(N & 3) && r < N) {
            const float4 v = *reinterpret_cast<const float4*>(S + r);
            s[4 * j] = v.x; s[4 * j + 1] = v.y; s[4 * j + 2] = v.z; s[4 * j + 3] = v.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[4 * j + e] = (live && r + e < N) ? S[r + e] : 0.0f;
        }
    }
}
template <int K>
__device__ __forceinline__ void rec_store_column(const float (&s)[K], float* __restrict__ S, int lane, int N) {
#pragma unroll
    for (int j = 0; j < K / 4; ++j) {
        const int r = rec_row(lane, 4 * j);
        if (!(N & 3) && r < N) {
            *reinterpret_cast<float4*>(S + r) = make_float4(s[4 * j], s[4 * j + 1], s[4 * j + 2], s[4 * j + 3]);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (r + e < N) S[r + e] = s[4 * j + e];
        }
    }
}

// a token's vector (K * REC_LANES numbers in shared memory, zero beyond the real ones) into the registers that match the column's
template <int K>
__device__ __forceinline__ void rec_load_vector(float (&v)[K], const float* __restrict__ row, int lane) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
#pragma unroll
    for (int j = 0; j < K / 4; ++j) {
        const float4 q = row4[lane + REC_LANES * j];
        v[4 * j] = q.x; v[4 * j + 1] = q.y; v[4 * j + 2] = q.z; v[4 * j + 3] = q.w;
    }
}

__device__ __forceinline__ float rec_group_sum(float v) {
#pragma unroll
    for (int o = REC_LANES / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ------------------------------------------------------------------------------------
// Causal convolution over time, one filter per channel:
//   y[t, c] = f(bias[c] + sum_j w[c, j] * x[t - (taps - 1) + j, c]),   f = silu or identity.
// x before this step's first token comes from the sequence's state, which holds its last taps - 1
// inputs (oldest first, [taps - 1][channels]; zero for a new sequence).
// Prompts: one kernel computes the outputs, a second one moves the states on (a thread per sequence
// and channel), because the outputs of a sequence's first tokens read the state that the update
// overwrites.  One token per sequence: a thread per (sequence, channel) does both.
// ------------------------------------------------------------------------------------
constexpr int CONV_TILE = 16;       // packed tokens a thread walks with its channel's last inputs in registers

// A thread takes one channel through CONV_TILE packed tokens: every input is read once (plus taps - 1 at the tile's
// start) and the window of the last inputs slides through registers.  Where the tile crosses into the next sequence
// the window is filled from that sequence's state.
__global__ void causal_conv_kernel(const float* __restrict__ proj, int splits, size_t split_stride, int cols, int col_off,
                                   int channels, const float* __restrict__ weight, const float* __restrict__ bias, int taps,
                                   int activation, const float* __restrict__ state, size_t slot_stride, float* __restrict__ out,
                                   const int* __restrict__ cu, const int* __restrict__ slots, int sequences, int n_tokens) {
    tt_pdl_launch_dependents();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int keep = taps - 1;
    float w[CONV_MAX_TAPS];
    float shift = 0.0f;
    if (c < channels) {                                          // filters are written by no kernel: fetched before the wait
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) w[j] = j < taps ? __ldg(weight + (size_t)c * taps + j) : 0.0f;
        shift = bias ? __ldg(bias + c) : 0.0f;
    }
    tt_pdl_wait();
    if (c >= channels) return;
    const int t0 = blockIdx.x * CONV_TILE, t1 = min(t0 + CONV_TILE, n_tokens);
    int b = tt_find_sequence(cu, sequences, t0);
    int first = cu[b], next = cu[b + 1];
    float win[CONV_MAX_TAPS];                                    // win[j], j < keep: the input (keep - j) tokens back
    auto fill = [&](int t) {                                     // the window as it stands before token t of sequence b
        const float* st = state + (size_t)slots[b] * slot_stride;
        const int i = t - first;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) {
            if (j < keep) {
                const int s = i - keep + j;
                win[j] = s >= 0 ? rec_sum_slices(proj + (size_t)(first + s) * cols + col_off + c, splits, split_stride)
                                : st[(size_t)(keep + s) * channels + c];
            }
        }
    };
    fill(t0);
    for (int t = t0; t < t1; ++t) {
        if (t == next) {                                         // the next sequence starts here
            ++b;
            first = next;
            next = cu[b + 1];
            fill(t);
        }
        const float x = rec_sum_slices(proj + (size_t)t * cols + col_off + c, splits, split_stride);
        float acc = shift;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
            if (j <= keep) acc = fmaf(w[j], j < keep ? win[j] : x, acc);     // oldest input first, the token's own last
        out[(size_t)t * channels + c] = activation ? rec_silu(acc) : acc;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
            if (j < keep) win[j] = j + 1 < keep ? win[j + 1] : x;
    }
}

// compute != 0: the sequence brings one token, whose output is computed here too
__global__ void causal_conv_state_kernel(const float* __restrict__ proj, int splits, size_t split_stride, int cols, int col_off,
                                         int channels, const float* __restrict__ weight, const float* __restrict__ bias, int taps,
                                         int activation, float* __restrict__ state, size_t slot_stride, float* __restrict__ out,
                                         const int* __restrict__ cu, const int* __restrict__ slots, int compute) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int b = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int first = cu[b], n = cu[b + 1] - first;
    if (n <= 0) return;
    float* st = state + (size_t)slots[b] * slot_stride;
    const int keep = taps - 1;
    float next[CONV_MAX_TAPS];
    // the last `keep` entries of (old state, then this step's inputs)
#pragma unroll
    for (int e = 0; e < CONV_MAX_TAPS; ++e) {
        if (e < keep) {
            const int idx = n + e;              // index into the concatenation
            next[e] = idx < keep ? st[(size_t)idx * channels + c]
                                 : rec_sum_slices(proj + (size_t)(first + idx - keep) * cols + col_off + c, splits, split_stride);
        }
    }
    if (compute) {
        float acc = bias ? __ldg(bias + c) : 0.0f;
        for (int j = 0; j < keep; ++j) acc = fmaf(__ldg(weight + (size_t)c * taps + j), st[(size_t)j * channels + c], acc);
        const float x = rec_sum_slices(proj + (size_t)first * cols + col_off + c, splits, split_stride);
        acc = fmaf(__ldg(weight + (size_t)c * taps + keep), x, acc);
        out[(size_t)first * channels + c] = activation ? rec_silu(acc) : acc;
    }
#pragma unroll
    for (int e = 0; e < CONV_MAX_TAPS; ++e)
        if (e < keep) st[(size_t)e * channels + c] = next[e];
}

extern "C" int tt_causal_conv(const float* proj, int splits, long long split_stride, int cols, int col_off, int channels,
                              const float* weight, const float* bias, int taps, int activation, float* state,
                              long long slot_stride, float* out, const int* cu, const int* slots, int sequences, int n_tokens,
                              int one_token_each, cudaStream_t stream) {
    if (n_tokens <= 0 || channels <= 0) return 0;
    const int threads = 128;
    const unsigned bx = (unsigned)((channels + threads - 1) / threads);
    if (taps < 1 || taps > CONV_MAX_TAPS || bx > 65535) return (int)cudaErrorInvalidValue;
    if (!one_token_each) {
        tt_launch_pdl(causal_conv_kernel, dim3((n_tokens + CONV_TILE - 1) / CONV_TILE, bx), dim3(threads), 0, stream, proj, splits, (size_t)split_stride, cols, col_off,
                      channels, weight, bias, taps, activation, (const float*)state, (size_t)slot_stride, out, cu, slots, sequences, n_tokens);
    }
    if (taps > 1 || one_token_each)
        tt_launch_pdl(causal_conv_state_kernel, dim3(sequences, bx), dim3(threads), 0, stream, proj, splits, (size_t)split_stride, cols,
                      col_off, channels, weight, bias, taps, activation, state, (size_t)slot_stride, out, cu, slots, one_token_each);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// Mamba-2 recurrence.  Per head h (group g = h / (heads / groups)), state S [N x P], token t:
//   dt = softplus(dt_raw[t, h] + dt_bias[h])            (no clamp)
//   S  = exp(-exp(A_log[h]) * dt) * S + dt * B[t, g] x[t, h]^T
//   y[t, h] = S^T C[t, g] + D[h] * x[t, h]
// xbc: float32 [tokens][inner + 2 * groups * N] (x, then B, then C: the convolution's output);
// dt_raw: column dt_col of the projection's partial sums; state: [slots][heads][P][N].
// ------------------------------------------------------------------------------------
// G column groups of REC_LANES lanes per CTA, each owning C neighbouring columns: (32, 1) gives a sequence the most
// warps (one long prompt, decoding); (16, 4) reads a token's vectors from shared memory once for four columns, which is
// what bounds the kernel once the grid fills the GPU (batches of prompts).
template <int K, int G, int C>
__global__ void __launch_bounds__(G* REC_LANES)
mamba2_scan_kernel(const float* __restrict__ xbc, int xbc_cols, const float* __restrict__ proj, int splits, size_t split_stride,
                   int cols, int dt_col, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                   const float* __restrict__ d_skip, float* __restrict__ state, float* __restrict__ y,
                   const int* __restrict__ cu, const int* __restrict__ slots, int heads, int P, int N, int groups, int chunk,
                   int vec, const float* __restrict__ fixed_decay) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ __align__(16) float rec_shared[];
    // two buffers of: B [chunk][NP], C [chunk][NP], x [chunk][TILE], decay [chunk], step [chunk]; rows are padded to
    // NP = K * REC_LANES numbers and the padding is zero, so the token loop needs no bounds
    constexpr int NP = K * REC_LANES, TILE = G * C;
    const int buffer_floats = 2 * chunk * NP + chunk * TILE + 2 * chunk;
    const int h = blockIdx.x, b = blockIdx.y, p0 = blockIdx.z * TILE;
    const int first = cu[b], n = cu[b + 1] - first;
    if (n <= 0) return;
    const int g = h / (heads / groups);
    const int inner = heads * P;
    const int lane = threadIdx.x % REC_LANES, col = (threadIdx.x / REC_LANES) * C;     // first of this group's columns in the tile
    const int width = min(TILE, P - p0);                        // columns of this tile that exist
    // fixed_decay: the head's decay is a constant and every step size is one (S = decay * S + B x^T, y = S^T C)
    const float fixed = fixed_decay ? __ldg(fixed_decay + h) : 0.0f;
    const float neg_a = fixed_decay ? 0.0f : -expf(__ldg(a_log + h)), bias = fixed_decay ? 0.0f : __ldg(dt_bias + h);
    const float skip = fixed_decay ? 0.0f : __ldg(d_skip + h);
    const bool vec_x = vec && (width & 3) == 0;

    auto stage = [&](int c0, float* base) {                      // asynchronous: B, C and x of tokens c0 .. of this sequence
        const int count = min(chunk, n - c0);
        const float* row = xbc + (size_t)(first + c0) * xbc_cols;
        rec_stage(base, NP, row + inner + g * N, xbc_cols, count, N, vec);
        rec_stage(base + chunk * NP, NP, row + inner + groups * N + g * N, xbc_cols, count, N, vec);
        rec_stage(base + 2 * chunk * NP, TILE, row + h * P + p0, xbc_cols, count, width, vec_x);
        rec_commit();
    };
    auto raw_step = [&](int c0) {                                // this thread's token of the chunk: the raw step size
        if (fixed_decay) return 0.0f;
        return rec_sum_slices(proj + (size_t)(first + c0 + threadIdx.x) * cols + dt_col + h, splits, split_stride);
    };
    auto put_scalars = [&](float* base, float raw) {
        const float dt = fixed_decay ? 1.0f : rec_softplus(raw + bias);
        base[2 * chunk * NP + chunk * TILE + threadIdx.x] = fixed_decay ? fixed : expf(neg_a * dt);
        base[2 * chunk * NP + chunk * TILE + chunk + threadIdx.x] = dt;
    };

    for (int e = threadIdx.x; e < 2 * buffer_floats; e += blockDim.x) rec_shared[e] = 0.0f;
    __syncthreads();
    stage(0, rec_shared);
    float* S = state + (((size_t)slots[b] * heads + h) * P + p0 + col) * N;          // column c of the group lies c * N further
    float s[C][K];
#pragma unroll
    for (int c = 0; c < C; ++c) rec_load_column<K>(s[c], S + (size_t)(p0 + col + c < P ? c : 0) * N, lane, N, p0 + col + c < P);
    if (threadIdx.x < min(chunk, n)) put_scalars(rec_shared, raw_step(0));
    int it = 0;
    for (int c0 = 0; c0 < n; c0 += chunk, ++it) {
        float* cur = rec_shared + (it & 1) * buffer_floats;
        float* nxt = rec_shared + ((it + 1) & 1) * buffer_floats;
        const int count = min(chunk, n - c0);
        const int count_next = min(chunk, n - c0 - chunk);       // <= 0: this is the last chunk
        float raw_next = 0.0f;
        if (count_next > 0) {
            stage(c0 + chunk, nxt);                              // lands while this chunk is worked on
            if (threadIdx.x < count_next) raw_next = raw_step(c0 + chunk);
            rec_wait<1>();
        } else {
            rec_wait<0>();
        }
        __syncthreads();
        const float* Bs = cur;
        const float* Cs = cur + chunk * NP;
        const float* xs = cur + 2 * chunk * NP;
        const float* decay = xs + chunk * TILE;
        const float* step = decay + chunk;
        for (int k = 0; k < count; ++k) {
            const float a = decay[k], dt = step[k];
            float bv[K], cv[K];                                  // all of the token's loads are asked for before the arithmetic
            rec_load_vector<K>(bv, Bs + k * NP, lane);
            rec_load_vector<K>(cv, Cs + k * NP, lane);
            float x[C], part[C];
#pragma unroll
            for (int c = 0; c < C; ++c) {
                x[c] = p0 + col + c < P ? xs[k * TILE + col + c] : 0.0f;
                const float dx = dt * x[c];
                float part0 = 0.0f, part1 = 0.0f;                // two chains, so that neighbouring rows do not wait for each other
#pragma unroll
                for (int i = 0; i < K; i += 2) {
                    s[c][i] = fmaf(dx, bv[i], a * s[c][i]);
                    part0 = fmaf(s[c][i], cv[i], part0);
                    s[c][i + 1] = fmaf(dx, bv[i + 1], a * s[c][i + 1]);
                    part1 = fmaf(s[c][i + 1], cv[i + 1], part1);
                }
                part[c] = part0 + part1;
            }
#pragma unroll
            for (int o = REC_LANES / 2; o > 0; o >>= 1) {        // the columns' sums over the lane group, side by side
#pragma unroll
                for (int c = 0; c < C; ++c) part[c] += __shfl_xor_sync(0xffffffffu, part[c], o);
            }
            if (lane == 0) {
#pragma unroll
                for (int c = 0; c < C; ++c)
                    if (p0 + col + c < P) y[(size_t)(first + c0 + k) * inner + h * P + p0 + col + c] = fmaf(skip, x[c], part[c]);
            }
        }
        if (count_next > 0 && threadIdx.x < count_next) put_scalars(nxt, raw_next);
        __syncthreads();                                         // this buffer may be filled again; the next one's scalars are written
    }
#pragma unroll
    for (int c = 0; c < C; ++c)
        if (p0 + col + c < P) rec_store_column<K>(s[c], S + (size_t)c * N, lane, N);
}

// Tokens staged at a time: 16 where two buffers of them fit the default 48 KB of shared memory, else 8.
static int rec_padded(int rows) { return rows <= 8 * REC_LANES ? 8 * REC_LANES : rows <= 16 * REC_LANES ? 16 * REC_LANES : 32 * REC_LANES; }
static int rec_chunk(int rows) { return rows <= 128 ? REC_CHUNK : REC_CHUNK / 2; }
static size_t rec_shared_bytes(int rows, int chunk, int tile) { return (size_t)2 * (2 * chunk * rec_padded(rows) + chunk * tile + 2 * chunk) * sizeof(float); }

constexpr int REC_WIDE_GROUPS = 16, REC_WIDE_COLS = 4;      // the form for grids that fill the GPU: 16 lane groups of 4 columns each

// Whether the grid of the (32, 1) form would fill the GPU more than twice over, so that the (16, 4) form pays
// (mode 0; 1 and 2 force the one or the other, for tests).  The wide form holds four columns of up to 128 rows.
static bool rec_wide(int mode, long long ctas, int rows) {
    if (rows > 16 * REC_LANES) return false;
    if (mode) return mode == 2;
    static int sms = 0;
    if (!sms) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
    }
    return ctas >= 2LL * sms;
}
static bool rec_aligned(const void* p, int a, int b, int c, int d) { return (((uintptr_t)p & 15) == 0) && !((a | b | c | d) & 3); }

static int mamba2_scan_launch(const float* xbc, int xbc_cols, const float* proj, int splits, long long split_stride, int cols,
                              int dt_col, const float* dt_bias, const float* a_log, const float* d_skip, float* state, float* y,
                              const int* cu, const int* slots, int sequences, int heads, int P, int N, int groups, int mode,
                              const float* fixed_decay, cudaStream_t stream) {
    if (sequences <= 0) return 0;
    if (N <= 0 || N > REC_MAX_ROWS || P <= 0 || groups <= 0 || heads % groups || sequences > 65535) return (int)cudaErrorInvalidValue;
    const int chunk = rec_chunk(N);
    const int vec = rec_aligned(xbc, xbc_cols, N, P, 0) ? 1 : 0;          // every row piece starts on 16 bytes
    const bool wide = rec_wide(mode, (long long)heads * sequences * ((P + REC_COLS - 1) / REC_COLS), N);
    const int tile = wide ? REC_WIDE_GROUPS * REC_WIDE_COLS : REC_COLS;
    const dim3 grid(heads, sequences, (P + tile - 1) / tile), block((wide ? REC_WIDE_GROUPS : REC_COLS) * REC_LANES);
    const size_t shared = rec_shared_bytes(N, chunk, tile);
#define TT_SCAN(K, G, C) tt_launch_pdl(mamba2_scan_kernel<K, G, C>, grid, block, shared, stream, xbc, xbc_cols, proj, splits, (size_t)split_stride, cols, dt_col, dt_bias, a_log, d_skip, state, y, cu, slots, heads, P, N, groups, chunk, vec, fixed_decay)
    if (wide) {
        if (N <= 8 * REC_LANES) TT_SCAN(8, REC_WIDE_GROUPS, REC_WIDE_COLS);
        else TT_SCAN(16, REC_WIDE_GROUPS, REC_WIDE_COLS);
    } else {
        if (N <= 8 * REC_LANES) TT_SCAN(8, REC_COLS, 1);
        else if (N <= 16 * REC_LANES) TT_SCAN(16, REC_COLS, 1);
        else TT_SCAN(32, REC_COLS, 1);
    }
#undef TT_SCAN
    TT_LAUNCH_CHECK();
}

extern "C" int tt_mamba2_scan(const float* xbc, int xbc_cols, const float* proj, int splits, long long split_stride, int cols,
                              int dt_col, const float* dt_bias, const float* a_log, const float* d_skip, float* state, float* y,
                              const int* cu, const int* slots, int sequences, int heads, int P, int N, int groups, int mode,
                              cudaStream_t stream) {
    return mamba2_scan_launch(xbc, xbc_cols, proj, splits, split_stride, cols, dt_col, dt_bias, a_log, d_skip, state, y, cu, slots,
                              sequences, heads, P, N, groups, mode, nullptr, stream);
}

// ------------------------------------------------------------------------------------
// Linear attention with a fixed decay per head: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, S [D x V] per head.
// It is the recurrence above with a constant decay, step size one, B = k, C = q, x = v and no skip, a group per head;
// vkq: float32 [tokens][heads * V + 2 * heads * D] (v, then k, then q: what tt_linear_attention_prepare writes);
// state: [slots][heads][V][D].
// ------------------------------------------------------------------------------------
extern "C" int tt_decay_scan(const float* vkq, int vkq_cols, const float* decay, float* state, float* out, const int* cu,
                             const int* slots, int sequences, int heads, int V, int D, int mode, cudaStream_t stream) {
    if (!decay) return (int)cudaErrorInvalidValue;
    return mamba2_scan_launch(vkq, vkq_cols, nullptr, 0, 0, 0, 0, nullptr, nullptr, nullptr, state, out, cu, slots, sequences, heads, V, D,
                              heads, mode, decay, stream);
}

// q, k and v of a linear attention from the partial sums of its input projection (columns [q | k | v | ...], q and k
// heads x D, v heads x V), as the scan reads them: [v | k | q].  activation != 0: silu on all three.  rotary_dim > 0:
// the first rotary_dim numbers of each head of q and k are rotated by the token's position (number i pairs with
// i + rotary_dim / 2, angle = position * inv_freq[i], float32).  k is multiplied by k_scale after the rotation.
__global__ void linear_attention_prepare_kernel(const float* __restrict__ proj, int splits, size_t split_stride, int cols, int heads,
                                                int D, int V, int activation, const float* __restrict__ inv_freq, int rotary_dim,
                                                float k_scale, float* __restrict__ vkq, const int* __restrict__ cu,
                                                const int* __restrict__ len_before, int sequences) {
    tt_pdl_launch_dependents();
    const int t = blockIdx.x;
    int pos = 0;
    if (rotary_dim > 0) {
        const int b = tt_find_sequence(cu, sequences, t);
        pos = len_before[b] + (t - cu[b]);
    }
    tt_pdl_wait();
    const int qk = heads * D, hv = heads * V;
    const float* row = proj + (size_t)t * cols;
    float* out = vkq + (size_t)t * (hv + 2 * qk);
    const int half = rotary_dim >> 1;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < 2 * qk + hv; j += gridDim.y * blockDim.x) {
        float x = rec_sum_slices(row + j, splits, split_stride);
        if (activation) x = rec_silu(x);
        if (j >= 2 * qk) {                                       // v
            out[j - 2 * qk] = x;
            continue;
        }
        const bool is_k = j >= qk;
        const int i = (is_k ? j - qk : j) % D;
        if (i < rotary_dim) {
            const int pair = i < half ? j + half : j - half;
            float other = rec_sum_slices(row + pair, splits, split_stride);
            if (activation) other = rec_silu(other);
            float sn, cs;
            sincosf((float)pos * __ldg(inv_freq + (i < half ? i : i - half)), &sn, &cs);
            x = i < half ? x * cs - other * sn : x * cs + other * sn;
        }
        if (is_k) out[hv + (j - qk)] = x * k_scale;
        else out[hv + qk + j] = x;
    }
}

extern "C" int tt_linear_attention_prepare(const float* proj, int splits, long long split_stride, int cols, int heads, int D, int V,
                                           int activation, const float* inv_freq, int rotary_dim, float k_scale, float* vkq,
                                           const int* cu, const int* len_before, int sequences, int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > D || (rotary_dim & 1) || 2 * heads * D + heads * V > cols) return (int)cudaErrorInvalidValue;
    const int total = 2 * heads * D + heads * V;
    const int want = n_tokens >= 1024 ? (total + 1023) / 1024 : (total + 255) / 256;                // few tokens: a token's columns over more blocks
    const int tiles = want < 32 ? want : 32;
    tt_launch_pdl(linear_attention_prepare_kernel, dim3(n_tokens, tiles), dim3(256), 0, stream, proj, splits, (size_t)split_stride, cols, heads, D,
                  V, activation, inv_freq, rotary_dim, k_scale, vkq, cu, len_before, sequences);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// Gated delta rule.  Per head h (query/key head g = h / (heads / qk_heads)), state S [D x V], token t:
//   q = q / sqrt(sum(q^2) + 1e-6) * D^-1/2,   k = k / sqrt(sum(k^2) + 1e-6)       (per head)
//   beta = sigmoid(b_raw[t, h]),   decay = exp(-exp(A_log[h]) * softplus(a_raw[t, h] + dt_bias[h]))
//   S = decay * S;  u = beta * (v - S^T k);  S = S + k u^T;  o[t, h] = S^T q
// qkv: float32 [tokens][2 * qk_heads * D + heads * V] (q, k, v: the convolutions' output); b_raw and
// a_raw: columns b_col + h and a_col + h of the projection's partial sums; state: [slots][heads][V][D].
// ------------------------------------------------------------------------------------
template <int K, int G, int C>
__global__ void __launch_bounds__(G* REC_LANES)
delta_scan_kernel(const float* __restrict__ qkv, int qkv_cols, const float* __restrict__ proj, int splits, size_t split_stride,
                  int cols, int b_col, int a_col, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                  float* __restrict__ state, float* __restrict__ o, const int* __restrict__ cu, const int* __restrict__ slots,
                  int heads, int qk_heads, int D, int V, int chunk, int vec) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ __align__(16) float rec_shared[];
    // two buffers of: q [chunk][DP], k [chunk][DP], v [chunk][TILE], decay [chunk], beta [chunk]; rows are padded to
    // DP = K * REC_LANES numbers and the padding is zero.  G lane groups of C neighbouring columns each, as in the kernel above.
    constexpr int DP = K * REC_LANES, TILE = G * C;
    const int buffer_floats = 2 * chunk * DP + chunk * TILE + 2 * chunk;
    const int h = blockIdx.x, b = blockIdx.y, p0 = blockIdx.z * TILE;
    const int first = cu[b], n = cu[b + 1] - first;
    if (n <= 0) return;
    const int g = h / (heads / qk_heads);
    const int lane = threadIdx.x % REC_LANES, col = (threadIdx.x / REC_LANES) * C;
    const int warp = threadIdx.x >> 5, wlane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int width = min(TILE, V - p0);
    const float neg_a = -expf(__ldg(a_log + h)), bias = __ldg(dt_bias + h), q_scale = rsqrtf((float)D);
    const int k_off = qk_heads * D, v_off = 2 * qk_heads * D;
    const bool vec_v = vec && (width & 3) == 0;

    auto stage = [&](int c0, float* base) {
        const int count = min(chunk, n - c0);
        const float* row = qkv + (size_t)(first + c0) * qkv_cols;
        rec_stage(base, DP, row + g * D, qkv_cols, count, D, vec);
        rec_stage(base + chunk * DP, DP, row + k_off + g * D, qkv_cols, count, D, vec);
        rec_stage(base + 2 * chunk * DP, TILE, row + v_off + h * V + p0, qkv_cols, count, width, vec_v);
        rec_commit();
    };
    auto raw_pair = [&](int c0) {                                // this thread's token of the chunk: raw write strength, raw decay input
        const float* row = proj + (size_t)(first + c0 + threadIdx.x) * cols;
        return make_float2(rec_sum_slices(row + b_col + h, splits, split_stride), rec_sum_slices(row + a_col + h, splits, split_stride));
    };
    auto put_scalars = [&](float* base, float2 raw) {
        base[2 * chunk * DP + chunk * TILE + threadIdx.x] = expf(neg_a * rec_softplus(raw.y + bias));
        base[2 * chunk * DP + chunk * TILE + chunk + threadIdx.x] = 1.0f / (1.0f + expf(-raw.x));
    };

    for (int e = threadIdx.x; e < 2 * buffer_floats; e += blockDim.x) rec_shared[e] = 0.0f;
    __syncthreads();
    stage(0, rec_shared);
    float* S = state + (((size_t)slots[b] * heads + h) * V + p0 + col) * D;
    float s[C][K];
#pragma unroll
    for (int c = 0; c < C; ++c) rec_load_column<K>(s[c], S + (size_t)(p0 + col + c < V ? c : 0) * D, lane, D, p0 + col + c < V);
    if (threadIdx.x < min(chunk, n)) put_scalars(rec_shared, raw_pair(0));
    int it = 0;
    for (int c0 = 0; c0 < n; c0 += chunk, ++it) {
        float* cur = rec_shared + (it & 1) * buffer_floats;
        float* nxt = rec_shared + ((it + 1) & 1) * buffer_floats;
        const int count = min(chunk, n - c0);
        const int count_next = min(chunk, n - c0 - chunk);
        float2 raw_next = make_float2(0.0f, 0.0f);
        if (count_next > 0) {
            stage(c0 + chunk, nxt);
            if (threadIdx.x < count_next) raw_next = raw_pair(c0 + chunk);
            rec_wait<1>();
        } else {
            rec_wait<0>();
        }
        __syncthreads();
        float* qs = cur;
        float* ks = cur + chunk * DP;
        // a warp per (token, q or k): sum of squares, scale to unit length (q also by D^-1/2)
        for (int item = warp; item < 2 * count; item += warps) {
            float* vecp = (item & 1 ? ks : qs) + (item >> 1) * DP;
            float sumsq = 0.0f;
            for (int r = wlane; r < D; r += 32) sumsq = fmaf(vecp[r], vecp[r], sumsq);
            const float scale = rsqrtf(tt_warp_sum(sumsq) + 1e-6f) * (item & 1 ? 1.0f : q_scale);
            for (int r = wlane; r < D; r += 32) vecp[r] *= scale;
        }
        __syncthreads();
        const float* vs = cur + 2 * chunk * DP;
        const float* decay = vs + chunk * TILE;
        const float* beta = decay + chunk;
        for (int k = 0; k < count; ++k) {
            const float a = decay[k], write = beta[k];
            float kv[K], qv[K];                                  // all of the token's loads are asked for before the arithmetic
            rec_load_vector<K>(kv, ks + k * DP, lane);
            rec_load_vector<K>(qv, qs + k * DP, lane);
            float part[C];
#pragma unroll
            for (int c = 0; c < C; ++c) {
                float part0 = 0.0f, part1 = 0.0f;
#pragma unroll
                for (int i = 0; i < K; i += 2) {
                    s[c][i] *= a;
                    part0 = fmaf(s[c][i], kv[i], part0);
                    s[c][i + 1] *= a;
                    part1 = fmaf(s[c][i + 1], kv[i + 1], part1);
                }
                part[c] = part0 + part1;
            }
#pragma unroll
            for (int o2 = REC_LANES / 2; o2 > 0; o2 >>= 1) {
#pragma unroll
                for (int c = 0; c < C; ++c) part[c] += __shfl_xor_sync(0xffffffffu, part[c], o2);
            }
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const float u = write * ((p0 + col + c < V ? vs[k * TILE + col + c] : 0.0f) - part[c]);
                float part0 = 0.0f, part1 = 0.0f;
#pragma unroll
                for (int i = 0; i < K; i += 2) {
                    s[c][i] = fmaf(kv[i], u, s[c][i]);
                    part0 = fmaf(s[c][i], qv[i], part0);
                    s[c][i + 1] = fmaf(kv[i + 1], u, s[c][i + 1]);
                    part1 = fmaf(s[c][i + 1], qv[i + 1], part1);
                }
                part[c] = part0 + part1;
            }
#pragma unroll
            for (int o2 = REC_LANES / 2; o2 > 0; o2 >>= 1) {
#pragma unroll
                for (int c = 0; c < C; ++c) part[c] += __shfl_xor_sync(0xffffffffu, part[c], o2);
            }
            if (lane == 0) {
#pragma unroll
                for (int c = 0; c < C; ++c)
                    if (p0 + col + c < V) o[(size_t)(first + c0 + k) * (heads * V) + h * V + p0 + col + c] = part[c];
            }
        }
        if (count_next > 0 && threadIdx.x < count_next) put_scalars(nxt, raw_next);
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < C; ++c)
        if (p0 + col + c < V) rec_store_column<K>(s[c], S + (size_t)c * D, lane, D);
}

extern "C" int tt_delta_scan(const float* qkv, int qkv_cols, const float* proj, int splits, long long split_stride, int cols,
                             int b_col, int a_col, const float* dt_bias, const float* a_log, float* state, float* o,
                             const int* cu, const int* slots, int sequences, int heads, int qk_heads, int D, int V, int mode,
                             cudaStream_t stream) {
    if (sequences <= 0) return 0;
    if (D <= 0 || D > REC_MAX_ROWS || V <= 0 || qk_heads <= 0 || heads % qk_heads || sequences > 65535) return (int)cudaErrorInvalidValue;
    const int chunk = rec_chunk(D);
    const int vec = rec_aligned(qkv, qkv_cols, D, V, 0) ? 1 : 0;
    const bool wide = rec_wide(mode, (long long)heads * sequences * ((V + REC_COLS - 1) / REC_COLS), D);
    const int tile = wide ? REC_WIDE_GROUPS * REC_WIDE_COLS : REC_COLS;
    const dim3 grid(heads, sequences, (V + tile - 1) / tile), block((wide ? REC_WIDE_GROUPS : REC_COLS) * REC_LANES);
    const size_t shared = rec_shared_bytes(D, chunk, tile);
#define TT_SCAN(K, G, C) tt_launch_pdl(delta_scan_kernel<K, G, C>, grid, block, shared, stream, qkv, qkv_cols, proj, splits, (size_t)split_stride, cols, b_col, a_col, dt_bias, a_log, state, o, cu, slots, heads, qk_heads, D, V, chunk, vec)
    if (wide) {
        if (D <= 8 * REC_LANES) TT_SCAN(8, REC_WIDE_GROUPS, REC_WIDE_COLS);
        else TT_SCAN(16, REC_WIDE_GROUPS, REC_WIDE_COLS);
    } else {
        if (D <= 8 * REC_LANES) TT_SCAN(8, REC_COLS, 1);
        else if (D <= 16 * REC_LANES) TT_SCAN(16, REC_COLS, 1);
        else TT_SCAN(32, REC_COLS, 1);
    }
#undef TT_SCAN
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// Gate and group norm behind a recurrence.  y: float32 [tokens][width], cut into groups of `group`
// neighbouring columns; gate: columns gate_col .. gate_col + width - 1 of a projection's partial sums.
//   gate_first != 0:  v = y * silu(gate);  out = v / sqrt(mean_group(v^2) + eps) * w
//   gate_first == 0:  out = y / sqrt(mean_group(y^2) + eps) * w * silu(gate)
// w (float32 [weight_len]) is indexed by column modulo weight_len: one weight for the whole width, or one
// per position inside a head that all heads share.  One block per (token, group).
// ------------------------------------------------------------------------------------
template <typename TOut>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, int width, int group, const float* __restrict__ proj,
                                        int splits, size_t split_stride, int cols, int gate_col,
                                        const float* __restrict__ weight, int weight_len, float eps, int gate_first,
                                        TOut* __restrict__ out, int gate_kind) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    __shared__ float reduce[32];
    const int groups = width / group;
    const int t = blockIdx.x / groups, gi = blockIdx.x - t * groups;
    const float* yr = y + (size_t)t * width + (size_t)gi * group;
    const float* gr = proj + (size_t)t * cols + gate_col + (size_t)gi * group;
    float sumsq = 0.0f;
    for (int j = threadIdx.x; j < group; j += blockDim.x) {
        float v = yr[j];
        if (gate_first) v *= rec_gate(rec_sum_slices(gr + j, splits, split_stride), gate_kind);
        sumsq += v * v;
    }
    const float r = rsqrtf(tt_block_sum(sumsq, reduce) / (float)group + eps);
    TOut* o = out + (size_t)t * width + (size_t)gi * group;
    for (int j = threadIdx.x; j < group; j += blockDim.x) {
        const float gate = rec_gate(rec_sum_slices(gr + j, splits, split_stride), gate_kind);
        const float w = __ldg(weight + (gi * group + j) % weight_len);
        const float v = gate_first ? yr[j] * gate * r * w : yr[j] * r * w * gate;
        o[j] = tt_from_float<TOut>(v);
    }
}

// The same with a group's numbers kept in registers between the two passes (up to GN_VALUES per thread), so every
// input is loaded once and all loads of a thread are in flight together: the form for groups of up to 8,192 numbers.
constexpr int GN_VALUES = 8;

template <typename TOut>
__global__ void __launch_bounds__(1024)
gated_group_norm_reg_kernel(const float* __restrict__ y, int width, int group, const float* __restrict__ proj, int splits,
                            size_t split_stride, int cols, int gate_col, const float* __restrict__ weight, int weight_len,
                            float eps, int gate_first, TOut* __restrict__ out, int gate_kind) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    __shared__ float reduce[32];
    const int groups = width / group;
    const int t = blockIdx.x / groups, gi = blockIdx.x - t * groups;
    const float* yr = y + (size_t)t * width + (size_t)gi * group;
    const float* gr = proj + (size_t)t * cols + gate_col + (size_t)gi * group;
    float v[GN_VALUES], gate[GN_VALUES];
    float sumsq = 0.0f;
#pragma unroll
    for (int e = 0; e < GN_VALUES; ++e) {
        const int j = threadIdx.x + e * blockDim.x;
        v[e] = 0.0f;
        gate[e] = 0.0f;
        if (j < group) {
            gate[e] = rec_gate(rec_sum_slices(gr + j, splits, split_stride), gate_kind);
            v[e] = gate_first ? yr[j] * gate[e] : yr[j];
            sumsq = fmaf(v[e], v[e], sumsq);
        }
    }
    const float r = rsqrtf(tt_block_sum(sumsq, reduce) / (float)group + eps);
    TOut* o = out + (size_t)t * width + (size_t)gi * group;
#pragma unroll
    for (int e = 0; e < GN_VALUES; ++e) {
        const int j = threadIdx.x + e * blockDim.x;
        if (j < group) {
            const float w = __ldg(weight + (gi * group + j) % weight_len);
            o[j] = tt_from_float<TOut>(gate_first ? v[e] * r * w : v[e] * r * w * gate[e]);
        }
    }
}

extern "C" int tt_gated_group_norm(const float* y, int n_tokens, int width, int group, const float* proj, int splits,
                                   long long split_stride, int cols, int gate_col, const float* weight, int weight_len, float eps,
                                   int gate_first, void* out, int out_dtype, int gate_kind, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (group <= 0 || width % group || weight_len <= 0) return (int)cudaErrorInvalidValue;
    const long long blocks = (long long)n_tokens * (width / group);
    if (blocks > 2147483647LL) return (int)cudaErrorInvalidValue;
    if (group <= 1024 * GN_VALUES) {
        int threads = (((group + 3) / 4 + 31) / 32) * 32;       // about four numbers a thread
        if (threads > 1024) threads = 1024;
        if (out_dtype == TT_F32)
            tt_launch_pdl(gated_group_norm_reg_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, y, width, group, proj, splits, (size_t)split_stride, cols, gate_col, weight, weight_len, eps, gate_first, (float*)out, gate_kind);
        else
            tt_launch_pdl(gated_group_norm_reg_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream, y, width, group, proj, splits, (size_t)split_stride, cols, gate_col, weight, weight_len, eps, gate_first, (__nv_bfloat16*)out, gate_kind);
        TT_LAUNCH_CHECK();
    }
    const int threads = group >= 2048 ? 256 : (group >= 256 ? 128 : (group > 32 ? 64 : 32));
    if (out_dtype == TT_F32)
        tt_launch_pdl(gated_group_norm_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, y, width, group, proj, splits, (size_t)split_stride, cols, gate_col, weight, weight_len, eps, gate_first, (float*)out, gate_kind);
    else
        tt_launch_pdl(gated_group_norm_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream, y, width, group, proj, splits, (size_t)split_stride, cols, gate_col, weight, weight_len, eps, gate_first, (__nv_bfloat16*)out, gate_kind);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// out[i] = wa * sum_s a[s][i] + wb * sum_s b[s][i]: two branches' outputs (each the partial sums of a
// product) weighted and added, float32.
// ------------------------------------------------------------------------------------
__global__ void weighted_pair_kernel(const float* __restrict__ a, int a_splits, size_t a_stride, float wa,
                                     const float* __restrict__ b, int b_splits, size_t b_stride, float wb,
                                     float* __restrict__ out, size_t total) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    out[i] = wa * rec_sum_slices(a + i, a_splits, a_stride) + wb * rec_sum_slices(b + i, b_splits, b_stride);
}

extern "C" int tt_weighted_pair(const float* a, int a_splits, long long a_stride, float wa, const float* b, int b_splits,
                                long long b_stride, float wb, float* out, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    const int threads = 256;
    tt_launch_pdl(weighted_pair_kernel, dim3((unsigned)((total + threads - 1) / threads)), dim3(threads), 0, stream, a, a_splits,
                  (size_t)a_stride, wa, b, b_splits, (size_t)b_stride, wb, out, (size_t)total);
    TT_LAUNCH_CHECK();
}
