// Kernels for layers that carry more per request than pages of keys and values: short causal filters over time with
// their tails, rotation of adjacent pairs over part of a head, values normalised before they are cached, a gated
// linear recurrence with a matrix state per head, and the element-wise pieces of a layer whose sublayers run side
// by side (tanh-GELU, per-head output gates, the gated residual sum).
//
// Storage is float or bfloat16 (template parameter), arithmetic float. Recurrent state, gates of the recurrence,
// norms, angles and the residual sum are float in both. With float storage these kernels are the 32-bit path.
//
// Every kernel takes a step's packed rows: tokens of several requests ("segments") one after the other, seg_start[s]
// the first row of segment s, seg_slot[s] the request's state slot. What a token's result depends on is its own
// request's earlier tokens and state only, and every reduction runs in an order fixed by the layer's sizes, so a
// result does not depend on how a prompt was cut or on what else is in the step.
#include "common.cuh"

IB_DEFINE_LAST_ERROR()

#define IB_LAUNCH(kernel, grid, block, smem, ...)                                                              \
    do {                                                                                                       \
        const int rc_ = ib::launch(#kernel, kernel, dim3(grid), dim3(block), size_t(smem), stream, 1u, __VA_ARGS__); \
        if (rc_) return rc_;                                                                                   \
    } while (0)

namespace {

using bf16 = __nv_bfloat16;

inline unsigned blocks_for(int64_t n, int threads) { return unsigned((n + threads - 1) / threads); }

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------------------------------------
// Short causal filter, per channel: y[t] = sum_j w[c, j] * u[t - (taps - 1) + j]. u before the first row of the
// step's segment comes from the request's tail (the last taps - 1 values of earlier steps, oldest first; zeros for a
// new request, which is what "nothing before the start" means). i_local is the token's index within its segment;
// `col` its channel's column in the rows, `tail` the channel's first tail value, tail_ld the channel count; the
// channel's tap j is w[j * w_stride].
template <typename T>
__device__ __forceinline__ float filtered(const T* __restrict__ rows, int64_t ld, int64_t t, int i_local, int col,
                                          const float* __restrict__ w, int64_t w_stride, int taps,
                                          const T* __restrict__ tail, int64_t tail_ld) {
    if (taps <= 1) {
        const float u = ib::to_f32(rows[t * ld + col]);
        return taps == 1 ? w[0] * u : u;
    }
    float y = 0.0f;
    for (int j = 0; j < taps; j++) {
        const int back = taps - 1 - j;
        const float u = i_local >= back ? ib::to_f32(rows[(t - back) * ld + col])
                                        : ib::to_f32(tail[int64_t(taps - 1 + i_local - back) * tail_ld]);
        y = fmaf(w[j * w_stride], u, y);
    }
    return y;
}

template <typename T>
__global__ void short_filter_kernel(const T* __restrict__ rows, int64_t ld, int col0, int channels,
                                    const float* __restrict__ w, int taps, const T* __restrict__ tails,
                                    const int* __restrict__ token_seg, const int* __restrict__ seg_start,
                                    const int* __restrict__ seg_slot, T* __restrict__ out, int64_t n_tokens) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * channels) return;
    const int64_t t = i / channels;
    const int c = int(i - t * channels);
    const int s = token_seg[t];
    const T* tail = tails ? tails + (int64_t(seg_slot[s]) * (taps - 1)) * channels + c : nullptr;
    out[i] = ib::from_f32<T>(filtered(rows, ld, t, int(t - seg_start[s]), col0 + c, w + int64_t(c) * taps, 1, taps, tail, channels));
}

// After a step: the tail of every segment's request becomes the last taps - 1 values of (old tail, the step's rows).
// One thread per (segment, channel) moves its values oldest first, reading ahead of what it writes.
template <typename T>
__global__ void filter_tail_kernel(const T* __restrict__ rows, int64_t ld, int col0, int channels, int taps,
                                   T* __restrict__ tails, const int* __restrict__ seg_start,
                                   const int* __restrict__ seg_slot) {
    ib::pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = blockIdx.y;
    if (c >= channels) return;
    const int keep = taps - 1;
    const int64_t t0 = seg_start[s];
    const int len = int(seg_start[s + 1] - t0);
    T* tail = tails + (int64_t(seg_slot[s]) * keep) * channels + c;
    for (int idx = 0; idx < keep; idx++) {
        const int src = len - keep + idx;
        tail[int64_t(idx) * channels] = src >= 0 ? rows[(t0 + src) * ld + col0 + c] : tail[int64_t(idx + len) * channels];
    }
}

// ------------------------------------------------------------------------------------------------
// From projected rows [q heads | k heads | v heads | ...] to what attention reads: optional short filter on every
// channel (its weights tap-major, filt_w[tap][channel], so that neighbouring channels' taps lie side by side), rotation of q and k, optional normalisation of v, q into q_out, k and v into the token's page.
// Rotation: channels (2i, 2i + 1) of a head, 2i < n_rot, turn by the angle of tables cos/sin [positions, n_rot / 2];
// the head's other channels stay.  v: each head divided by sqrt(mean(v^2) + eps), no weight.
// One warp per (token, head of q, k or v); a lane keeps up to PREP_PAIRS pairs of a head in registers.
constexpr int PREP_PAIRS = 4;           // heads of up to 64 * PREP_PAIRS channels

template <typename T>
__global__ void __launch_bounds__(128)
qkv_prepare_kernel(const T* __restrict__ rows, int64_t ld, int col_base, int inline_tail,
                   const float* __restrict__ filt_w, int taps, T* tails, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                   int n_rot, int norm_v, float eps, const int* __restrict__ positions,
                   const int* __restrict__ token_seg, const int* __restrict__ seg_start,
                   const int* __restrict__ seg_slot, const int* __restrict__ block_table, int64_t max_blocks,
                   T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache, int64_t n_tokens,
                   int n_heads, int n_kv, int d, int dv, int page_size, int write_cache, int64_t n_pages, int* status) {
    ib::pdl_wait();
    const int lane = threadIdx.x & 31;
    const int units = n_heads + 2 * n_kv;
    const int64_t wi = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wi >= n_tokens * units) return;
    const int64_t t = wi / units;
    const int u = int(wi - t * units);
    const int kind = u < n_heads ? 0 : (u < n_heads + n_kv ? 1 : 2);            // q, k, v
    const int head = kind == 0 ? u : (kind == 1 ? u - n_heads : u - n_heads - n_kv);
    const int width = kind == 2 ? dv : d;
    const int col0 = kind == 0 ? head * d : (kind == 1 ? n_heads * d + head * d : (n_heads + n_kv) * d + head * dv);
    const int channels = (n_heads + n_kv) * d + n_kv * dv;
    const int s = token_seg[t];
    const int i_local = int(t - seg_start[s]);
    const int pos = positions[t];
    const bool filt = filt_w != nullptr && taps > 0;
    const T* tail = filt && taps > 1 ? tails + (int64_t(seg_slot[s]) * (taps - 1)) * channels : nullptr;

    float a[PREP_PAIRS], b[PREP_PAIRS];
    float ss = 0.0f;
#pragma unroll
    for (int r = 0; r < PREP_PAIRS; r++) {
        const int p = lane + 32 * r;
        a[r] = b[r] = 0.0f;
        if (2 * p < width) {
            const int c = col0 + 2 * p;                          // channel; its column in the rows is col_base + c
            const bool two = 2 * p + 1 < width;                  // (a head of odd size ends with half a pair)
            if (filt) {
                a[r] = filtered(rows, ld, t, i_local, col_base + c, filt_w + c, channels, taps, tail + c, channels);
                if (two) b[r] = filtered(rows, ld, t, i_local, col_base + c + 1, filt_w + c + 1, channels, taps, tail + c + 1, channels);
                if (inline_tail && taps > 1) {
                    // one token per request: this lane is the only reader of the two channels' tails; it moves them
                    T* tw = tails + (int64_t(seg_slot[s]) * (taps - 1)) * channels + c;
                    for (int idx = 0; idx + 1 < taps - 1; idx++) {
                        tw[int64_t(idx) * channels] = tw[int64_t(idx + 1) * channels];
                        if (two) tw[int64_t(idx) * channels + 1] = tw[int64_t(idx + 1) * channels + 1];
                    }
                    tw[int64_t(taps - 2) * channels] = rows[t * ld + col_base + c];
                    if (two) tw[int64_t(taps - 2) * channels + 1] = rows[t * ld + col_base + c + 1];
                }
            } else {
                a[r] = ib::to_f32(rows[t * ld + col_base + c]);
                if (two) b[r] = ib::to_f32(rows[t * ld + col_base + c + 1]);
            }
            if (kind != 2 && cos_t && 2 * p < n_rot) {
                const float cs = cos_t[int64_t(pos) * (n_rot / 2) + p], sn = sin_t[int64_t(pos) * (n_rot / 2) + p];
                const float ra = a[r] * cs - b[r] * sn;
                const float rb = b[r] * cs + a[r] * sn;
                a[r] = ra;
                b[r] = rb;
            }
            ss = fmaf(a[r], a[r], ss);
            ss = fmaf(b[r], b[r], ss);
        }
    }
    if (kind == 2 && norm_v) {
        ss = ib::warp_sum(ss);
        const float f = rsqrtf(ss / float(width) + eps);
#pragma unroll
        for (int r = 0; r < PREP_PAIRS; r++) {
            a[r] *= f;
            b[r] *= f;
        }
    }
    T* dst;
    if (kind == 0) {
        dst = q_out + (t * n_heads + head) * d;
    } else {
        if (!write_cache) return;
        const int page = block_table[int64_t(s) * max_blocks + pos / page_size];
        if (page < 0 || page >= n_pages) {
            if (status && lane == 0) atomicExch(status, 2);
            return;
        }
        dst = (kind == 1 ? k_cache : v_cache) + ((int64_t(page) * n_kv + head) * page_size + pos % page_size) * width;
    }
#pragma unroll
    for (int r = 0; r < PREP_PAIRS; r++) {
        const int p = lane + 32 * r;
        if (2 * p < width) {
            dst[2 * p] = ib::from_f32<T>(a[r]);
            if (2 * p + 1 < width) dst[2 * p + 1] = ib::from_f32<T>(b[r]);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// ctx[t, h, :] *= sigmoid(gate[t, h]); the gate logits are columns gate_col .. gate_col + heads of the rows.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ ctx, const T* __restrict__ rows, int64_t ld, int gate_col,
                                 int64_t n_tokens, int n_heads, int dv) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * n_heads * dv) return;
    const int64_t th = i / dv;
    const int64_t t = th / n_heads;
    const int h = int(th - t * n_heads);
    const float g = sigmoidf_(ib::to_f32(rows[t * ld + gate_col + h]));
    ctx[i] = ib::from_f32<T>(ib::to_f32(ctx[i]) * g);
}

// ------------------------------------------------------------------------------------------------
// tanh-GELU: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
// Input: columns [col0, col0 + width) of rows with leading dimension ld; output contiguous [tokens, width].
template <typename T>
__global__ void gelu_tanh_kernel(const T* __restrict__ x, int64_t ld, int col0, int64_t width, T* __restrict__ out, int64_t n) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t t = i / width;
    const float z = ib::to_f32(x[t * ld + col0 + (i - t * width)]);
    out[i] = ib::from_f32<T>(0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))));
}

// ------------------------------------------------------------------------------------------------
// out = x + sigmoid(g1) * (a * p + b * q) + sigmoid(g2) * r, all float [tokens, width]; the gate logits are columns
// [0, width) and [width, 2 width) of rows `gates` with leading dimension ldg. q, r (and then g2) may be absent; with
// gates absent the terms are added as they are.
__global__ void gated_sum_kernel(const float* x, const float* __restrict__ gates, int64_t ldg,
                                 const float* __restrict__ p, float a, const float* __restrict__ q, float b,
                                 const float* __restrict__ r, float* out, int64_t n_tokens, int64_t width) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * width) return;
    const int64_t t = i / width, c = i - t * width;
    float m = a * p[i];
    if (q) m = fmaf(b, q[i], m);
    float y = gates ? sigmoidf_(gates[t * ldg + c]) * m : m;
    if (r) y += gates ? sigmoidf_(gates[t * ldg + width + c]) * r[i] : r[i];
    out[i] = x[i] + y;
}

// ------------------------------------------------------------------------------------------------
// Gated linear recurrence with a matrix state per head (the forget gate also weighs what is written):
//   f = low + (1 - low) * sigmoid(f_raw),  q = silu(q_raw)
//   S <- diag(f) S + (1 - f) v^T          S [d, dv] float, per request and head, kept in `state` between steps
//   o = S^T q,  out = o / sqrt(mean(o^2) + eps) * norm_w      (per head; norm_w [dv] shared by the heads)
// Rows `proj` are float [tokens, ld] with q_raw at q_col, f_raw at f_col (both heads * d wide) and v at v_col
// (heads * dv wide).
//
// A CTA walks over the tokens of one segment, in order, for one head and `cb` of its columns. Thread (kg, col) keeps
// MAXK rows of column col of S in registers (rows kg * kpt ..; kpt <= MAXK, the rest padded with zeros); tokens are
// staged `chunk` at a time in shared memory as [token][kg][MAXK], so that the inner loop is 16-byte loads and three
// floating-point operations per state element; the column sums over kg are added in ascending order.
// Two ways to run it, with the same arithmetic per element and therefore the same bits:
//   * one CTA per (segment, head) over all columns, gates computed while staging, the head's norm at the end of every
//     chunk: one launch, for steps of a few tokens per request;
//   * a grid over column blocks as well, for prompt portions: the chain over the tokens is the critical path, so the
//     columns of a head are spread over many SMs. The gates are then computed once by recurrence_gates_kernel (in
//     place, instead of once per column block), the CTAs write the bare o, and head_norm_kernel normalises.
__device__ __forceinline__ float silu_value(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float forget_value(float low, float x) { return __fmaf_rn(1.0f - low, sigmoidf_(x), low); }

__global__ void recurrence_gates_kernel(float* __restrict__ proj, int64_t ld, int q_col, int f_col,
                                        const float* __restrict__ lower, int64_t n_tokens, int width) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * width) return;
    const int64_t t = i / width;
    const int c = int(i - t * width);
    float* row = proj + t * ld;
    row[q_col + c] = silu_value(row[q_col + c]);
    row[f_col + c] = forget_value(lower[c], row[f_col + c]);
}

// One warp per (token, head): out = o / sqrt(mean(o^2) + eps) * w, lanes striding over the columns.
template <typename TOut>
__global__ void head_norm_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps,
                                 TOut* __restrict__ out, int64_t n_rows, int dv) {
    ib::pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t r = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const float* x = o + r * dv;
    float ss = 0.0f;
    for (int j = lane; j < dv; j += 32) ss = fmaf(x[j], x[j], ss);
    ss = ib::warp_sum(ss);
    const float f = rsqrtf(ss / float(dv) + eps);
    for (int j = lane; j < dv; j += 32) out[r * dv + j] = ib::from_f32<TOut>(x[j] * f * w[j]);
}

// One chunk of staged tokens through a thread's share of the state: the arithmetic of both forms of the kernel.
// qs, fs: [token][ks][MAXK] (stride kstride); vs: [token][cb]; part: [token][ks][cb].
template <int MAXK>
__device__ __forceinline__ void recurrence_chunk(float (&S)[MAXK], const float* __restrict__ qs, const float* __restrict__ fs,
                                                 const float* __restrict__ vs, float* __restrict__ part, int n, int kstride,
                                                 int kg, int ks, int cb, int col_l) {
#pragma unroll 4
    for (int c = 0; c < n; c++) {
        const float v = vs[c * cb + col_l];
        const float4* f4 = reinterpret_cast<const float4*>(fs + c * kstride + kg * MAXK);
        const float4* q4 = reinterpret_cast<const float4*>(qs + c * kstride + kg * MAXK);
        // four partial sums (rows 4i, 4i+1, 4i+2, 4i+3), added pairwise at the end: a chain of MAXK / 4 instead of MAXK
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
        for (int k4 = 0; k4 < MAXK / 4; k4++) {
            const float4 f = f4[k4], q = q4[k4];
            S[4 * k4 + 0] = fmaf(f.x, S[4 * k4 + 0], (1.0f - f.x) * v);
            S[4 * k4 + 1] = fmaf(f.y, S[4 * k4 + 1], (1.0f - f.y) * v);
            S[4 * k4 + 2] = fmaf(f.z, S[4 * k4 + 2], (1.0f - f.z) * v);
            S[4 * k4 + 3] = fmaf(f.w, S[4 * k4 + 3], (1.0f - f.w) * v);
            a0 = fmaf(S[4 * k4 + 0], q.x, a0);
            a1 = fmaf(S[4 * k4 + 1], q.y, a1);
            a2 = fmaf(S[4 * k4 + 2], q.z, a2);
            a3 = fmaf(S[4 * k4 + 3], q.w, a3);
        }
        part[(c * ks + kg) * cb + col_l] = (a0 + a1) + (a2 + a3);
    }
}

__device__ __forceinline__ void copy16_async(float* smem_dst, const float* gmem_src) {
    const uint32_t d = uint32_t(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}

template <typename TOut, int MAXK>
__global__ void __launch_bounds__(MAXK > 8 ? 512 : 1024)
gated_recurrence_kernel(const float* __restrict__ proj, int64_t ld, int q_col, int f_col, int v_col,
                        const float* __restrict__ lower, const float* __restrict__ norm_w, float eps,
                        float* __restrict__ state, const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                        TOut* __restrict__ out, float* __restrict__ raw_out, int n_heads, int d, int dv, int ks, int kpt,
                        int cb, int chunk, int activated, int write_state, int pipelined) {
    ib::pdl_wait();
    extern __shared__ __align__(16) float sm[];
    const int kstride = ks * MAXK;               // staged rows: [kg][MAXK]; a padded row f = 0 keeps a state row at zero
    const int n_buf = pipelined ? 2 : 1;
    float* qs = sm;                              // [n_buf][chunk][ks][MAXK]
    float* fs = qs + n_buf * chunk * kstride;
    float* vs = fs + n_buf * chunk * kstride;    // [n_buf][chunk][cb]
    float* part = vs + n_buf * chunk * cb;       // [chunk][ks][cb]
    float* os = part + chunk * ks * cb;          // [chunk][cb] (the form with the norm inside only)
    const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
    const int col_l = tid % cb, kg = tid / cb;
    const int col0 = blockIdx.z * cb;
    const int col = col0 + col_l;
    const bool active = kg < ks && col < dv;
    const int k0 = kg * kpt;
    const int nk = active ? max(0, min(kpt, d - k0)) : 0;
    const int64_t t0 = seg_start[s];
    const int len = int(seg_start[s + 1] - t0);
    float* S_g = state + (int64_t(seg_slot[s]) * n_heads + h) * int64_t(d) * dv;
    float S[MAXK];
#pragma unroll
    for (int kk = 0; kk < MAXK; kk++) S[kk] = kk < nk ? S_g[int64_t(k0 + kk) * dv + col] : 0.0f;

    if (pipelined) {
        // Prompt portions, gates already applied, d = ks * MAXK, every column offset a multiple of four floats: the
        // rows are copied as they lie, 16 bytes per asynchronous copy, one chunk ahead of the one being computed.
        const int q4 = d / 4, v4 = cb / 4;
        auto request = [&](int c0, int b) {
            const int n = min(chunk, len - c0);
            for (int idx = tid; idx < n * q4; idx += blockDim.x) {
                const int c = idx / q4, j = (idx - c * q4) * 4;
                const float* row = proj + (t0 + c0 + c) * ld;
                copy16_async(qs + (b * chunk + c) * kstride + j, row + q_col + h * d + j);
                copy16_async(fs + (b * chunk + c) * kstride + j, row + f_col + h * d + j);
            }
            for (int idx = tid; idx < n * v4; idx += blockDim.x) {
                const int c = idx / v4, j = (idx - c * v4) * 4;
                if (col0 + j < dv)
                    copy16_async(vs + (b * chunk + c) * cb + j, proj + (t0 + c0 + c) * ld + v_col + h * dv + col0 + j);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        request(0, 0);
        int b = 0;
        for (int c0 = 0; c0 < len; c0 += chunk, b ^= 1) {
            const int n = min(chunk, len - c0);
            if (c0 + chunk < len) {
                request(c0 + chunk, b ^ 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();                     // the chunk has arrived; the last chunk's sums have been read
            if (active)
                recurrence_chunk<MAXK>(S, qs + b * chunk * kstride, fs + b * chunk * kstride, vs + b * chunk * cb, part, n,
                                       kstride, kg, ks, cb, col_l);
            __syncthreads();
            for (int idx = tid; idx < n * cb; idx += blockDim.x) {
                const int c = idx / cb, j = idx - c * cb;
                float o = 0.0f;
                for (int g = 0; g < ks; g++) o += part[(c * ks + g) * cb + j];
                if (col0 + j < dv) raw_out[((t0 + c0 + c) * n_heads + h) * int64_t(dv) + col0 + j] = o;
            }
        }
    } else {
        for (int c0 = 0; c0 < len; c0 += chunk) {
            const int n = min(chunk, len - c0);
            for (int idx = tid; idx < n * kstride; idx += blockDim.x) {
                const int c = idx / kstride, r = idx - c * kstride;
                const int g = r / MAXK, kk = r - g * MAXK;
                const int k = g * kpt + kk;
                float q = 0.0f, f = 0.0f;
                if (kk < kpt && k < d) {
                    const float* row = proj + (t0 + c0 + c) * ld;
                    q = row[q_col + h * d + k];
                    f = row[f_col + h * d + k];
                    if (!activated) {
                        q = silu_value(q);
                        f = forget_value(lower[h * d + k], f);
                    }
                }
                qs[idx] = q;
                fs[idx] = f;
            }
            for (int idx = tid; idx < n * cb; idx += blockDim.x) {
                const int c = idx / cb, j = col0 + (idx - c * cb);
                vs[idx] = j < dv ? proj[(t0 + c0 + c) * ld + v_col + h * dv + j] : 0.0f;
            }
            __syncthreads();
            if (active) recurrence_chunk<MAXK>(S, qs, fs, vs, part, n, kstride, kg, ks, cb, col_l);
            __syncthreads();
            for (int idx = tid; idx < n * cb; idx += blockDim.x) {
                const int c = idx / cb, j = idx - c * cb;
                float o = 0.0f;
                for (int g = 0; g < ks; g++) o += part[(c * ks + g) * cb + j];
                if (raw_out) {
                    if (col0 + j < dv) raw_out[((t0 + c0 + c) * n_heads + h) * int64_t(dv) + col0 + j] = o;
                } else {
                    os[idx] = o;
                }
            }
            __syncthreads();
            if (!raw_out) {
                for (int c = warp; c < n; c += n_warps) {
                    float ss = 0.0f;
                    for (int j = lane; j < dv; j += 32) ss = fmaf(os[c * cb + j], os[c * cb + j], ss);
                    ss = ib::warp_sum(ss);
                    const float f = rsqrtf(ss / float(dv) + eps);
                    TOut* o = out + ((t0 + c0 + c) * n_heads + h) * int64_t(dv);
                    for (int j = lane; j < dv; j += 32) o[j] = ib::from_f32<TOut>(os[c * cb + j] * f * norm_w[j]);
                }
                __syncthreads();
            }
        }
    }
    if (write_state) {
#pragma unroll
        for (int kk = 0; kk < MAXK; kk++)
            if (kk < nk) S_g[int64_t(k0 + kk) * dv + col] = S[kk];
    }
}


// ------------------------------------------------------------------------------------------------
// The same three for bfloat16 rows whose sizes and addresses allow 16-byte accesses (8 values a thread).
__device__ __forceinline__ void unpack8(const uint4& u, float (&x)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(h[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}

__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    return u;
}

__global__ void gelu_tanh_vec_kernel(const bf16* __restrict__ x, int64_t ld, int col0, int64_t width8, bf16* __restrict__ out,
                                     int64_t n8) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const int64_t t = i / width8, j = i - t * width8;
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(x + t * ld + col0 + j * 8), v);
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const float z = v[e];
        v[e] = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    }
    *reinterpret_cast<uint4*>(out + i * 8) = pack8(v);
}

__global__ void head_gate_vec_kernel(bf16* __restrict__ ctx, const bf16* __restrict__ rows, int64_t ld, int gate_col,
                                     int64_t n8, int n_heads, int dv8) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const int64_t th = i / dv8;
    const int64_t t = th / n_heads;
    const int h = int(th - t * n_heads);
    const float g = sigmoidf_(__bfloat162float(rows[t * ld + gate_col + h]));
    float v[8];
    uint4* p = reinterpret_cast<uint4*>(ctx + i * 8);
    unpack8(*p, v);
#pragma unroll
    for (int e = 0; e < 8; e++) v[e] *= g;
    *p = pack8(v);
}

// V bfloat16 values (V = 4 or 8) as one 8- or 16-byte access.
template <int V> struct VecOf;
template <> struct VecOf<8> { using type = uint4; };
template <> struct VecOf<4> { using type = uint2; };

template <int V>
__device__ __forceinline__ void load_bf16(const bf16* p, float (&x)[V]) {
    const typename VecOf<V>::type u = *reinterpret_cast<const typename VecOf<V>::type*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < V / 2; i++) {
        const float2 f = __bfloat1622float2(h[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}

template <int V>
__device__ __forceinline__ void store_bf16(bf16* p, const float (&x)[V]) {
    typename VecOf<V>::type u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < V / 2; i++) h[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    *reinterpret_cast<typename VecOf<V>::type*>(p) = u;
}

// One warp per (token, head of q, k or v); lane l takes channels V l .. V l + V - 1 of the head: V = 4 for heads of up
// to 128 channels (every lane of a 128-wide head has work), V = 8 for heads of up to 256.
template <int V>
__global__ void __launch_bounds__(128)
qkv_prepare_vec_kernel(const bf16* __restrict__ rows, int64_t ld, int col_base, int inline_tail,
                       const float* __restrict__ filt_w, int taps, bf16* tails, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, int n_rot, int norm_v, float eps,
                       const int* __restrict__ positions, const int* __restrict__ token_seg,
                       const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                       const int* __restrict__ block_table, int64_t max_blocks, bf16* __restrict__ q_out,
                       bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int64_t n_tokens, int n_heads, int n_kv,
                       int d, int dv, int page_size, int write_cache, int64_t n_pages, int* status) {
    ib::pdl_wait();
    using Vec = typename VecOf<V>::type;
    const int lane = threadIdx.x & 31;
    const int units = n_heads + 2 * n_kv;
    const int64_t wi = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wi >= n_tokens * units) return;
    const int64_t t = wi / units;
    const int u = int(wi - t * units);
    const int kind = u < n_heads ? 0 : (u < n_heads + n_kv ? 1 : 2);
    const int head = kind == 0 ? u : (kind == 1 ? u - n_heads : u - n_heads - n_kv);
    const int width = kind == 2 ? dv : d;
    const int col0 = kind == 0 ? head * d : (kind == 1 ? n_heads * d + head * d : (n_heads + n_kv) * d + head * dv);
    const int channels = (n_heads + n_kv) * d + n_kv * dv;
    const int s = token_seg[t];
    const int i_local = int(t - seg_start[s]);
    const int pos = positions[t];
    const bool mine = V * lane < width;
    const int c = col0 + V * lane;                               // first of this lane's channels
    float x[V];
#pragma unroll
    for (int e = 0; e < V; e++) x[e] = 0.0f;
    if (mine) {
        if (filt_w != nullptr && taps > 0) {
            bf16* tail = taps > 1 ? tails + (int64_t(seg_slot[s]) * (taps - 1)) * channels + c : nullptr;
            for (int j = 0; j < taps; j++) {
                const int back = taps - 1 - j;
                const bf16* src = i_local >= back ? rows + (t - back) * ld + col_base + c
                                                  : tail + int64_t(taps - 1 + i_local - back) * channels;
                float uv[V];
                load_bf16<V>(src, uv);
                const float4* w4 = reinterpret_cast<const float4*>(filt_w + int64_t(j) * channels + c);
#pragma unroll
                for (int e4 = 0; e4 < V / 4; e4++) {
                    const float4 w = w4[e4];
                    x[4 * e4 + 0] = fmaf(w.x, uv[4 * e4 + 0], x[4 * e4 + 0]);
                    x[4 * e4 + 1] = fmaf(w.y, uv[4 * e4 + 1], x[4 * e4 + 1]);
                    x[4 * e4 + 2] = fmaf(w.z, uv[4 * e4 + 2], x[4 * e4 + 2]);
                    x[4 * e4 + 3] = fmaf(w.w, uv[4 * e4 + 3], x[4 * e4 + 3]);
                }
            }
            if (inline_tail && taps > 1) {
                for (int idx = 0; idx + 1 < taps - 1; idx++)
                    *reinterpret_cast<Vec*>(tail + int64_t(idx) * channels) = *reinterpret_cast<const Vec*>(tail + int64_t(idx + 1) * channels);
                *reinterpret_cast<Vec*>(tail + int64_t(taps - 2) * channels) = *reinterpret_cast<const Vec*>(rows + t * ld + col_base + c);
            }
        } else {
            load_bf16<V>(rows + t * ld + col_base + c, x);
        }
        if (kind != 2 && cos_t) {
#pragma unroll
            for (int i = 0; i < V / 2; i++) {
                const int p = (V / 2) * lane + i;
                if (2 * p < n_rot) {
                    const float cs = cos_t[int64_t(pos) * (n_rot / 2) + p], sn = sin_t[int64_t(pos) * (n_rot / 2) + p];
                    const float ra = x[2 * i] * cs - x[2 * i + 1] * sn;
                    const float rb = x[2 * i + 1] * cs + x[2 * i] * sn;
                    x[2 * i] = ra;
                    x[2 * i + 1] = rb;
                }
            }
        }
    }
    if (kind == 2 && norm_v) {
        float ss = 0.0f;
#pragma unroll
        for (int e = 0; e < V; e++) ss = fmaf(x[e], x[e], ss);
        ss = ib::warp_sum(ss);
        const float f = rsqrtf(ss / float(width) + eps);
#pragma unroll
        for (int e = 0; e < V; e++) x[e] *= f;
    }
    if (!mine) return;
    bf16* dst;
    if (kind == 0) {
        dst = q_out + (t * n_heads + head) * d;
    } else {
        if (!write_cache) return;
        const int page = block_table[int64_t(s) * max_blocks + pos / page_size];
        if (page < 0 || page >= n_pages) {
            if (status && lane == 0) atomicExch(status, 2);
            return;
        }
        dst = (kind == 1 ? k_cache : v_cache) + ((int64_t(page) * n_kv + head) * page_size + pos % page_size) * width;
    }
    store_bf16<V>(dst + V * lane, x);
}

}  // namespace

// ================================================================================================
// C entry points. dtype arguments: 0 = float, 1 = bfloat16.

IB_EXPORT int ib_short_filter(const void* rows, int64_t ld, int col0, int channels, const float* w, int taps,
                              const void* tails, const int* token_seg, const int* seg_start, const int* seg_slot,
                              void* out, int64_t n_tokens, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || channels <= 0) return IB_OK;
    if (taps < 1 || (taps > 1 && !tails)) return ib::fail(IB_ERR_ARG, "ib_short_filter: taps %d, or no tails", taps);
    const int64_t n = n_tokens * channels;
    if (dtype == IB_F32)
        IB_LAUNCH(short_filter_kernel<float>, blocks_for(n, 256), 256, 0, (const float*)rows, ld, col0, channels, w, taps,
                  (const float*)tails, token_seg, seg_start, seg_slot, (float*)out, n_tokens);
    else if (dtype == IB_BF16)
        IB_LAUNCH(short_filter_kernel<bf16>, blocks_for(n, 256), 256, 0, (const bf16*)rows, ld, col0, channels, w, taps,
                  (const bf16*)tails, token_seg, seg_start, seg_slot, (bf16*)out, n_tokens);
    else
        return ib::fail(IB_ERR_ARG, "ib_short_filter: unknown dtype %d", dtype);
    return ib::check_launch("ib_short_filter");
}

IB_EXPORT int ib_filter_tail(const void* rows, int64_t ld, int col0, int channels, int taps, void* tails,
                             const int* seg_start, const int* seg_slot, int n_segments, int dtype, cudaStream_t stream) {
    if (n_segments <= 0 || channels <= 0 || taps <= 1) return IB_OK;
    if (n_segments > 65535) return ib::fail(IB_ERR_ARG, "ib_filter_tail: too many segments");
    const dim3 grid{blocks_for(channels, 128), unsigned(n_segments), 1u};
    if (dtype == IB_F32)
        IB_LAUNCH(filter_tail_kernel<float>, grid, 128, 0, (const float*)rows, ld, col0, channels, taps, (float*)tails, seg_start, seg_slot);
    else if (dtype == IB_BF16)
        IB_LAUNCH(filter_tail_kernel<bf16>, grid, 128, 0, (const bf16*)rows, ld, col0, channels, taps, (bf16*)tails, seg_start, seg_slot);
    else
        return ib::fail(IB_ERR_ARG, "ib_filter_tail: unknown dtype %d", dtype);
    return ib::check_launch("ib_filter_tail");
}

// The widest head (keys or values) that ib_qkv_prepare takes.
IB_EXPORT int ib_qkv_prepare_max_head_dim() { return 64 * PREP_PAIRS; }

IB_EXPORT int ib_qkv_prepare(const void* rows, int64_t ld, int col_base, int inline_tail, const float* filt_w, int taps, void* tails,
                             const float* cos_t, const float* sin_t, int n_rot, int norm_v, float eps,
                             const int* positions, const int* token_seg, const int* seg_start, const int* seg_slot,
                             const int* block_table, int64_t max_blocks, void* q_out, void* k_cache, void* v_cache,
                             int64_t n_tokens, int n_heads, int n_kv, int d, int dv, int page_size, int write_cache,
                             int64_t n_pages, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (d <= 0 || dv <= 0 || d > 64 * PREP_PAIRS || dv > 64 * PREP_PAIRS)
        return ib::fail(IB_ERR_ARG, "ib_qkv_prepare: head sizes %d / %d must be at most %d", d, dv, 64 * PREP_PAIRS);
    if (n_rot < 0 || n_rot % 2 || n_rot > d) return ib::fail(IB_ERR_ARG, "ib_qkv_prepare: %d rotated channels of %d", n_rot, d);
    if (filt_w && taps > 1 && !tails) return ib::fail(IB_ERR_ARG, "ib_qkv_prepare: a filter of %d taps needs tails", taps);
    if (n_heads <= 0 || n_kv <= 0 || page_size <= 0) return ib::fail(IB_ERR_ARG, "ib_qkv_prepare: bad sizes");
    const int64_t warps = n_tokens * (n_heads + 2 * n_kv);
    if (dtype == IB_F32)
        IB_LAUNCH(qkv_prepare_kernel<float>, blocks_for(warps, 4), 128, 0, (const float*)rows, ld, col_base, inline_tail, filt_w, taps, (float*)tails, cos_t, sin_t,
                  n_rot, norm_v, eps, positions, token_seg, seg_start, seg_slot, block_table, max_blocks, (float*)q_out,
                  (float*)k_cache, (float*)v_cache, n_tokens, n_heads, n_kv, d, dv, page_size, write_cache, n_pages, status);
    else if (dtype == IB_BF16 && d % 8 == 0 && dv % 8 == 0 && ld % 8 == 0 && col_base % 8 == 0 &&
             !((uintptr_t(rows) | uintptr_t(tails) | uintptr_t(q_out) | uintptr_t(k_cache) | uintptr_t(v_cache) | uintptr_t(filt_w)) & 15))
    {
        // (chosen by sizes and addresses, never by the number of rows)
        if (d <= 128 && dv <= 128)
            IB_LAUNCH(qkv_prepare_vec_kernel<4>, blocks_for(warps, 4), 128, 0, (const bf16*)rows, ld, col_base, inline_tail, filt_w, taps, (bf16*)tails, cos_t, sin_t,
                      n_rot, norm_v, eps, positions, token_seg, seg_start, seg_slot, block_table, max_blocks, (bf16*)q_out,
                      (bf16*)k_cache, (bf16*)v_cache, n_tokens, n_heads, n_kv, d, dv, page_size, write_cache, n_pages, status);
        else
            IB_LAUNCH(qkv_prepare_vec_kernel<8>, blocks_for(warps, 4), 128, 0, (const bf16*)rows, ld, col_base, inline_tail, filt_w, taps, (bf16*)tails, cos_t, sin_t,
                      n_rot, norm_v, eps, positions, token_seg, seg_start, seg_slot, block_table, max_blocks, (bf16*)q_out,
                      (bf16*)k_cache, (bf16*)v_cache, n_tokens, n_heads, n_kv, d, dv, page_size, write_cache, n_pages, status);
    }
    else if (dtype == IB_BF16)
        IB_LAUNCH(qkv_prepare_kernel<bf16>, blocks_for(warps, 4), 128, 0, (const bf16*)rows, ld, col_base, inline_tail, filt_w, taps, (bf16*)tails, cos_t, sin_t,
                  n_rot, norm_v, eps, positions, token_seg, seg_start, seg_slot, block_table, max_blocks, (bf16*)q_out,
                  (bf16*)k_cache, (bf16*)v_cache, n_tokens, n_heads, n_kv, d, dv, page_size, write_cache, n_pages, status);
    else
        return ib::fail(IB_ERR_ARG, "ib_qkv_prepare: unknown dtype %d", dtype);
    return ib::check_launch("ib_qkv_prepare");
}

IB_EXPORT int ib_head_gate(void* ctx, const void* rows, int64_t ld, int gate_col, int64_t n_tokens, int n_heads, int dv,
                           int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    const int64_t n = n_tokens * n_heads * dv;
    if (dtype == IB_F32)
        IB_LAUNCH(head_gate_kernel<float>, blocks_for(n, 256), 256, 0, (float*)ctx, (const float*)rows, ld, gate_col, n_tokens, n_heads, dv);
    else if (dtype == IB_BF16 && dv % 8 == 0 && !(uintptr_t(ctx) & 15))
        IB_LAUNCH(head_gate_vec_kernel, blocks_for(n / 8, 256), 256, 0, (bf16*)ctx, (const bf16*)rows, ld, gate_col, n / 8, n_heads, dv / 8);
    else if (dtype == IB_BF16)
        IB_LAUNCH(head_gate_kernel<bf16>, blocks_for(n, 256), 256, 0, (bf16*)ctx, (const bf16*)rows, ld, gate_col, n_tokens, n_heads, dv);
    else
        return ib::fail(IB_ERR_ARG, "ib_head_gate: unknown dtype %d", dtype);
    return ib::check_launch("ib_head_gate");
}

IB_EXPORT int ib_gelu_tanh(const void* x, int64_t ld, int col0, int64_t width, void* out, int64_t n_tokens, int dtype,
                           cudaStream_t stream) {
    const int64_t n = n_tokens * width;
    if (n <= 0) return IB_OK;
    if (dtype == IB_F32)
        IB_LAUNCH(gelu_tanh_kernel<float>, blocks_for(n, 256), 256, 0, (const float*)x, ld, col0, width, (float*)out, n);
    else if (dtype == IB_BF16 && width % 8 == 0 && ld % 8 == 0 && col0 % 8 == 0 && !((uintptr_t(x) | uintptr_t(out)) & 15))
        IB_LAUNCH(gelu_tanh_vec_kernel, blocks_for(n / 8, 256), 256, 0, (const bf16*)x, ld, col0, width / 8, (bf16*)out, n / 8);
    else if (dtype == IB_BF16)
        IB_LAUNCH(gelu_tanh_kernel<bf16>, blocks_for(n, 256), 256, 0, (const bf16*)x, ld, col0, width, (bf16*)out, n);
    else
        return ib::fail(IB_ERR_ARG, "ib_gelu_tanh: unknown dtype %d", dtype);
    return ib::check_launch("ib_gelu_tanh");
}

IB_EXPORT int ib_gated_sum(const float* x, const float* gates, int64_t ldg, const float* p, float a, const float* q,
                           float b, const float* r, float* out, int64_t n_tokens, int64_t width, cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0) return IB_OK;
    if (!p) return ib::fail(IB_ERR_ARG, "ib_gated_sum: the first term is missing");
    IB_LAUNCH(gated_sum_kernel, blocks_for(n_tokens * width, 256), 256, 0, x, gates, ldg, p, a, q, b, r, out, n_tokens, width);
    return ib::check_launch("ib_gated_sum");
}

// How the rows of a head's state are shared among threads: ks threads per column with kpt rows each. As many threads
// as a CTA over all columns may have (1024, or 512 where a thread keeps more than 8 rows), so that a thread's share
// is short; the choice depends on (d, dv) only. Returns false if the head does not fit.
static bool recurrence_split(int d, int dv, int* ks, int* kpt) {
    if (d <= 0 || dv <= 0 || dv > 1024) return false;
    int k = 1024 / dv;
    k = k > d ? d : k;
    int per = (d + k - 1) / k;
    if (per > 8) {
        k = 512 / dv;
        if (k < 1) return false;
        k = k > d ? d : k;
        per = (d + k - 1) / k;
        if (per > 32) return false;
    }
    k = (d + per - 1) / per;                       // no thread group without rows
    *ks = k;
    *kpt = per;
    return true;
}

// 1 if a head's state of d x dv fits the recurrence kernel's registers, else 0.
IB_EXPORT int ib_gated_recurrence_fits(int d, int dv) {
    int ks, kpt;
    return recurrence_split(d, dv, &ks, &kpt) ? 1 : 0;
}

template <typename TOut, int MAXK>
static int launch_recurrence(dim3 grid, int threads, size_t smem, cudaStream_t stream, const float* proj, int64_t ld,
                             int q_col, int f_col, int v_col, const float* lower, const float* norm_w, float eps,
                             float* state, const int* seg_start, const int* seg_slot, TOut* out, float* raw_out,
                             int n_heads, int d, int dv, int ks, int kpt, int cb, int chunk, int activated, int write_state,
                             int pipelined) {
    IB_LAUNCH((gated_recurrence_kernel<TOut, MAXK>), grid, threads, smem, proj, ld, q_col, f_col, v_col, lower, norm_w, eps,
              state, seg_start, seg_slot, out, raw_out, n_heads, d, dv, ks, kpt, cb, chunk, activated, write_state, pipelined);
    return ib::check_launch("ib_gated_recurrence");
}

// `spread` 0: one CTA per (segment, head), one launch. `spread` 1 (prompt portions): gates in place first, then CTAs
// per column block that write the bare o into `scratch` (float [tokens, heads * dv]), then the heads' norm.
// proj is overwritten by the gates in that case. sm_count sizes the column blocks.
IB_EXPORT int ib_gated_recurrence(float* proj, int64_t ld, int q_col, int f_col, int v_col, const float* lower,
                                  const float* norm_w, float eps, float* state, const int* seg_start,
                                  const int* seg_slot, void* out, int n_segments, int n_heads, int d, int dv,
                                  int write_state, int out_dtype, cudaStream_t stream, int spread, float* scratch,
                                  int64_t n_tokens, int sm_count, int col_block) {
    if (n_segments <= 0) return IB_OK;
    int ks, kpt;
    if (n_heads <= 0 || n_heads > 65535 || !recurrence_split(d, dv, &ks, &kpt))
        return ib::fail(IB_ERR_ARG, "ib_gated_recurrence: %d heads with a state of %d x %d do not fit", n_heads, d, dv);
    if (out_dtype != IB_F32 && out_dtype != IB_BF16) return ib::fail(IB_ERR_ARG, "ib_gated_recurrence: unknown output dtype %d", out_dtype);
    const int maxk = kpt <= 8 ? 8 : 32;
    int cb = dv;
    int pipelined = 0;
    if (spread) {
        if (!scratch || n_tokens <= 0) return ib::fail(IB_ERR_ARG, "ib_gated_recurrence: the spread form needs scratch rows");
        // Column blocks: the chain over a segment's tokens is the critical path, so a head's columns are spread over
        // CTAs of at least 128 threads (a warp per scheduler) until there is about one CTA per SM.
        const int units = n_segments * n_heads, sms = sm_count > 0 ? sm_count : 148;
        while (cb % 8 == 0 && ks * (cb / 2) >= 128 && units * ((dv + cb / 2 - 1) / (cb / 2)) <= sms) cb /= 2;
        if (col_block > 0 && col_block <= dv && col_block % 4 == 0) cb = col_block;      // (for measurements)
        pipelined = d == ks * maxk && kpt == maxk && d % 4 == 0 && cb % 4 == 0 && dv % 4 == 0 && ld % 4 == 0 && q_col % 4 == 0 &&
                    f_col % 4 == 0 && v_col % 4 == 0 && !(uintptr_t(proj) & 15);
        IB_LAUNCH(recurrence_gates_kernel, blocks_for(n_tokens * n_heads * d, 256), 256, 0, proj, ld, q_col, f_col, lower, n_tokens, n_heads * d);
    }
    const int blocks_z = (dv + cb - 1) / cb;
    const int threads = (ks * cb + 31) / 32 * 32;
    const int n_buf = pipelined ? 2 : 1;
    const int per_token = n_buf * (2 * ks * maxk + cb) + ks * cb + (spread ? 0 : cb);
    int chunk = 11264 / per_token;                           // 44 KB of staging at most
    chunk = chunk < 1 ? 1 : (chunk > 16 ? 16 : chunk);
    const size_t smem = size_t(chunk) * per_token * sizeof(float);
    if (smem > 48 * 1024) return ib::fail(IB_ERR_ARG, "ib_gated_recurrence: a token of %d floats does not fit the staging area", per_token);
    const dim3 grid{unsigned(n_segments), unsigned(n_heads), unsigned(blocks_z)};
    float* raw = spread ? scratch : nullptr;
    int rc;
#define IB_REC(TOUT, MK)                                                                                                 \
    rc = launch_recurrence<TOUT, MK>(grid, threads, smem, stream, proj, ld, q_col, f_col, v_col, lower, norm_w, eps, state, \
                                     seg_start, seg_slot, (TOUT*)out, raw, n_heads, d, dv, ks, kpt, cb, chunk, spread, write_state, pipelined)
    if (out_dtype == IB_F32) {
        if (maxk == 8) IB_REC(float, 8); else IB_REC(float, 32);
    } else {
        if (maxk == 8) IB_REC(bf16, 8); else IB_REC(bf16, 32);
    }
#undef IB_REC
    if (rc) return rc;
    if (spread) {
        const int64_t rows = n_tokens * n_heads;
        if (out_dtype == IB_F32)
            IB_LAUNCH(head_norm_kernel<float>, blocks_for(rows, 8), 256, 0, (const float*)scratch, norm_w, eps, (float*)out, rows, dv);
        else
            IB_LAUNCH(head_norm_kernel<bf16>, blocks_for(rows, 8), 256, 0, (const float*)scratch, norm_w, eps, (bf16*)out, rows, dv);
        return ib::check_launch("ib_gated_recurrence");
    }
    return IB_OK;
}
