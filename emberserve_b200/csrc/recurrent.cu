// Mixers that carry state of fixed size from token to token instead of a growing cache:
//
//  * a matrix memory per head, S_t = a_t S_(t-1) + b_t k_t v_t^T, read as o_t = S_t^T q_t.  With a
//    constant decay per head and b = 1 this is linear ("lightning") attention; with gates a_t, b_t
//    from an exponential-gating recurrence and a normaliser vector n_t = a_t n_(t-1) + b_t k_t it is
//    the matrix memory of the mLSTM (Beck et al., "xLSTM: Extended Long Short-Term Memory");
//  * the stabilised gates of that memory (ems_mlstm_gates);
//  * a gated diagonal recurrence per channel, S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t (the
//    real-gated linear recurrent unit of De et al., "Griffin: Mixing Gated Linear Recurrences with
//    Local Attention for Efficient Language Models");
//  * the norm-and-gate step that follows a memory read (ems_group_norm_gate).
//
// Everything that enters a recurrence is 32-bit: states, decays, gates, the products with the state.
// The projections q, k, v, u, y arrive in the activation type and are widened once.  A request's
// tokens are walked in order by the same code whether they come as a prompt, a portion or alone, so
// a position's result does not depend on the cut.  States live in slots [slot, ...] of a float
// tensor; a block reads the state of its request's slot, runs the step's tokens and writes it back.
#include "common.cuh"

namespace ems {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
// log(sigmoid(z)) = min(z, 0) - log(1 + exp(-|z|))
__device__ __forceinline__ float logsigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// input activations of the memory's q, k, v
#define EMS_IN_NONE 0
#define EMS_IN_SILU 1
__device__ __forceinline__ float in_act(float z, int act) { return act == EMS_IN_SILU ? z * sigmoid_f(z) : z; }

// ---------------------------------------------------------------------------------------
// matrix memory

constexpr int MR_TT = 16;     // tokens staged per tile
constexpr int MR_COLS = 64;   // value columns per block (8 warps x 8 columns)
constexpr int MR_SLICES = 4;  // lanes that share a column: each holds every fourth row of S

struct MatRecParams {
    const void* q; const void* k; const void* v;   // [N, ld*] views; head h begins at column h * D (h * V)
    long long ldq, ldk, ldv;
    const float* decay_head;    // [H] constant decay per head, or null
    const float* a;             // [N, H] decay of every token (used when decay_head is null)
    const float* b;             // [N, H] input scale of every token, or null (= 1)
    const float* denom_floor;   // [N, H] with the normaliser: denom = max(|n.q|, floor) + denom_eps
    float* denom;               // [N, H] out (normaliser only)
    float* state;               // [slots, H, head_stride]: S [D, V] then, with the normaliser, n [D]
    const int* slots;           // [rows]
    const int* cu_q;            // [rows + 1]
    float* out;                 // [N, H * V] float
    int H, D, V, head_stride, normaliser, act;
    float q_scale, denom_eps;
};

template <typename T, int DPT>
__global__ void __launch_bounds__(256) matrix_recurrence_kernel(const MatRecParams p) {
    extern __shared__ float smem[];
    const int D = p.D, V = p.V;
    float* qs = smem;                    // [TT][D]
    float* ks = qs + MR_TT * D;          // [TT][D]   (already times b_t)
    float* vs = ks + MR_TT * D;          // [TT][MR_COLS]
    float* as = vs + MR_TT * MR_COLS;    // [TT]
    const int row = blockIdx.z, head = blockIdx.y;
    const int q0 = p.cu_q[row], qlen = p.cu_q[row + 1] - q0;
    if (qlen <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slice = lane & (MR_SLICES - 1), colw = lane >> 2;
    const int lcol = warp * 8 + colw;                  // column inside the block
    const int col = blockIdx.x * MR_COLS + lcol;       // column of [v | 1]
    const int ncols = V + (p.normaliser ? 1 : 0);
    const bool live = col < ncols;
    const bool is_norm = p.normaliser && col == V;
    float* st = p.state + ((size_t)p.slots[row] * p.H + head) * p.head_stride;

    float S[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = i * MR_SLICES + slice;
        S[i] = (live && d < D) ? (is_norm ? st[(size_t)D * V + d] : st[(size_t)d * V + col]) : 0.f;
    }
    const T* qg = reinterpret_cast<const T*>(p.q);
    const T* kg = reinterpret_cast<const T*>(p.k);
    const T* vg = reinterpret_cast<const T*>(p.v);
    const float decay_const = p.decay_head ? p.decay_head[head] : 1.f;

    for (int t0 = 0; t0 < qlen; t0 += MR_TT) {
        const int cnt = min(MR_TT, qlen - t0);
        __syncthreads();  // the tile before is consumed
        for (int idx = threadIdx.x; idx < cnt * D; idx += blockDim.x) {
            const int t = idx / D, d = idx % D;
            const size_t tok = (size_t)(q0 + t0 + t);
            const float bt = p.b ? p.b[tok * p.H + head] : 1.f;
            qs[t * D + d] = in_act(to_f32<T>(qg[tok * p.ldq + (size_t)head * D + d]), p.act) * p.q_scale;
            ks[t * D + d] = in_act(to_f32<T>(kg[tok * p.ldk + (size_t)head * D + d]), p.act) * bt;
        }
        for (int idx = threadIdx.x; idx < cnt * MR_COLS; idx += blockDim.x) {
            const int t = idx / MR_COLS, c = idx % MR_COLS;
            const int gc = blockIdx.x * MR_COLS + c;
            const size_t tok = (size_t)(q0 + t0 + t);
            float val = 0.f;
            if (gc < V) val = in_act(to_f32<T>(vg[tok * p.ldv + (size_t)head * V + gc]), p.act);
            else if (p.normaliser && gc == V) val = 1.f;
            vs[t * MR_COLS + c] = val;
        }
        if (threadIdx.x < cnt) {
            const size_t tok = (size_t)(q0 + t0 + threadIdx.x);
            as[threadIdx.x] = p.decay_head ? decay_const : p.a[tok * p.H + head];
        }
        __syncthreads();
        for (int t = 0; t < cnt; ++t) {
            const float a = as[t];
            const float vj = vs[t * MR_COLS + lcol];
            const float* kr = ks + t * D;
            const float* qr = qs + t * D;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < DPT; ++i) {
                const int d = i * MR_SLICES + slice;
                if (d < D) {
                    S[i] = fmaf(a, S[i], kr[d] * vj);
                    acc = fmaf(S[i], qr[d], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (live && slice == 0) {
                const size_t tok = (size_t)(q0 + t0 + t);
                if (is_norm)
                    p.denom[tok * p.H + head] = fmaxf(fabsf(acc), p.denom_floor[tok * p.H + head]) + p.denom_eps;
                else
                    p.out[tok * ((size_t)p.H * V) + (size_t)head * V + col] = acc;
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = i * MR_SLICES + slice;
            if (d < D) {
                if (is_norm) st[(size_t)D * V + d] = S[i];
                else st[(size_t)d * V + col] = S[i];
            }
        }
    }
}

template <typename T>
static int launch_matrix_recurrence(const MatRecParams& p, int rows, cudaStream_t stream) {
    const int ncols = p.V + (p.normaliser ? 1 : 0);
    const dim3 grid((ncols + MR_COLS - 1) / MR_COLS, p.H, rows);
    int threads = 32 * ((min(ncols, MR_COLS) + 7) / 8);
    const size_t smem = sizeof(float) * ((size_t)MR_TT * (2 * p.D + MR_COLS) + MR_TT);
    if (smem > 48 * 1024) return EMS_ERR_SHAPE;
    const int need = (p.D + MR_SLICES - 1) / MR_SLICES;
    if (need <= 8) matrix_recurrence_kernel<T, 8><<<grid, threads, smem, stream>>>(p);
    else if (need <= 16) matrix_recurrence_kernel<T, 16><<<grid, threads, smem, stream>>>(p);
    else if (need <= 32) matrix_recurrence_kernel<T, 32><<<grid, threads, smem, stream>>>(p);
    else if (need <= 64) matrix_recurrence_kernel<T, 64><<<grid, threads, smem, stream>>>(p);
    else return EMS_ERR_SHAPE;
    return launch_status();
}

// ---------------------------------------------------------------------------------------
// the gates of the mLSTM: log input gate i = cap tanh(x_i / cap), log forget gate f =
// logsigmoid(cap tanh(x_f / cap)), running maximum m_t = max(f + m_(t-1), i) (m starts at 0 in a
// fresh slot), a_t = exp(f + m_(t-1) - m_t), b_t = exp(i - m_t), floor_t = exp(-m_t).
// One warp per (request, head): the lanes take 32 tokens' transcendental work side by side, the
// maximum runs through them in order.

__global__ void mlstm_gates_kernel(const float* __restrict__ pre, const void* __restrict__ bias_i,
                                   const void* __restrict__ bias_f, int b_dtype, float cap,
                                   float* __restrict__ state, int head_stride, int m_offset,
                                   const int* __restrict__ slots, const int* __restrict__ cu_q, int rows, int H,
                                   float* __restrict__ a_out, float* __restrict__ b_out,
                                   float* __restrict__ floor_out) {
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= rows * H) return;
    const int row = unit / H, head = unit % H, lane = threadIdx.x & 31;
    const int q0 = cu_q[row], qlen = cu_q[row + 1] - q0;
    if (qlen <= 0) return;
    float* mp = state + ((size_t)slots[row] * H + head) * head_stride + m_offset;
    float m = *mp;
    const float bi = load_any(bias_i, b_dtype, head), bf = load_any(bias_f, b_dtype, head);
    for (int t0 = 0; t0 < qlen; t0 += 32) {
        const int cnt = min(32, qlen - t0);
        float ig = 0.f, fg = 0.f;
        if (lane < cnt) {
            const size_t tok = (size_t)(q0 + t0 + lane);
            const float xi = pre[tok * 2 * H + head] + bi, xf = pre[tok * 2 * H + H + head] + bf;
            ig = cap > 0.f ? cap * tanhf(xi / cap) : xi;
            fg = logsigmoid_f(cap > 0.f ? cap * tanhf(xf / cap) : xf);
        }
        float before = 0.f, after = 0.f;
        for (int j = 0; j < cnt; ++j) {
            const float fj = __shfl_sync(0xffffffffu, fg, j), ij = __shfl_sync(0xffffffffu, ig, j);
            const float m_new = fmaxf(fj + m, ij);
            if (lane == j) { before = m; after = m_new; }
            m = m_new;
        }
        if (lane < cnt) {
            const size_t at = (size_t)(q0 + t0 + lane) * H + head;
            a_out[at] = expf(fg + before - after);
            b_out[at] = expf(ig - after);
            floor_out[at] = expf(-after);
        }
    }
    if (lane == 0) *mp = m;
}

// ---------------------------------------------------------------------------------------
// what follows a memory read: o / denom (per token and group, optional), RMS norm of each of
// `groups` equal consecutive parts of the row, gain, sigmoid gate.  out = rms(o / denom) * w * sigmoid(g).
// One warp per (token, group); a block per (token, group) when a group is long.

template <typename T, bool BLOCK>
__global__ void group_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ denom,
                                       const void* __restrict__ w, int w_dtype, const T* __restrict__ gate,
                                       long long ldg, T* __restrict__ out, int N, int C, int groups, float eps) {
    __shared__ float red[33];
    const int gs = C / groups;
    int unit, lane, width;
    if (BLOCK) { unit = blockIdx.x; lane = threadIdx.x; width = blockDim.x; }
    else { unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); lane = threadIdx.x & 31; width = 32; }
    if (unit >= N * groups) return;   // (whole warps, or the whole block, leave together)
    const int tok = unit / groups, g = unit % groups;
    const float inv_den = denom ? 1.f / denom[(size_t)tok * groups + g] : 1.f;
    const float* src = o + (size_t)tok * C + (size_t)g * gs;
    float ss = 0.f;
    for (int c = lane; c < gs; c += width) {
        const float x = src[c] * inv_den;
        ss = fmaf(x, x, ss);
    }
    ss = BLOCK ? block_sum(ss, red) : warp_sum(ss);
    const float r = rsqrtf(ss / gs + eps) * inv_den;
    for (int c = lane; c < gs; c += width) {
        const int ch = g * gs + c;
        float y = src[c] * r * load_any(w, w_dtype, ch);
        if (gate) y *= sigmoid_f(to_f32<T>(gate[(size_t)tok * ldg + ch]));
        out[(size_t)tok * C + ch] = from_f32<T>(y);
    }
}

// ---------------------------------------------------------------------------------------
// the gated diagonal recurrence.  A thread owns (request, channel).  Gate pre-activations arrive
// as [2, blocks, N, C / blocks] float (r then i; the layout that one batched product per gate over
// the blocks of a block-diagonal matrix leaves): r = sigmoid(pre_r + br), i = sigmoid(pre_i + bi),
// log a = -c r softplus(lam), S = a S + sqrt(1 - a^2) i u, out = S * gelu_tanh(y).

template <typename T>
__global__ void rglru_scan_kernel(const T* __restrict__ u, const float* __restrict__ pre,
                                  const void* __restrict__ br, const void* __restrict__ bi,
                                  const void* __restrict__ lam, int p_dtype, const T* __restrict__ y, long long ldy,
                                  int y_act, float cmul, float* __restrict__ state, const int* __restrict__ slots,
                                  const int* __restrict__ cu_q, T* __restrict__ out, int N, int C, int blocks) {
    const int row = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int q0 = cu_q[row], qlen = cu_q[row + 1] - q0;
    if (qlen <= 0) return;
    const int bw = C / blocks, blk = c / bw, j = c % bw;
    const float rb = load_any(br, p_dtype, c), ib = load_any(bi, p_dtype, c);
    const float sp = cmul * softplus_f(load_any(lam, p_dtype, c));
    float* sp_state = state + (size_t)slots[row] * C + c;
    float S = *sp_state;
    const float* pr = pre + ((size_t)blk * N + q0) * bw + j;   // the r gate; the i gate lies N * C further
    const size_t gate_i = (size_t)N * C;
#pragma unroll 4
    for (int t = 0; t < qlen; ++t) {
        const size_t tok = (size_t)(q0 + t);
        const float r = sigmoid_f(pr[(size_t)t * bw] + rb);
        const float ig = sigmoid_f(pr[(size_t)t * bw + gate_i] + ib);
        const float log_a = -sp * r;
        const float a = expf(log_a);
        const float mult = sqrtf(-expm1f(2.f * log_a));   // sqrt(1 - a^2) without the cancellation
        S = fmaf(a, S, mult * ig * to_f32<T>(u[tok * C + c]));
        float yy = to_f32<T>(y[tok * ldy + c]);
        if (y_act) yy = gelu_tanh_f(yy);
        out[tok * C + c] = from_f32<T>(S * yy);
    }
    *sp_state = S;
}

}  // namespace ems

using namespace ems;

EMS_EXPORT int ems_matrix_recurrence(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                     long long ldv, int dtype, int act, float q_scale, const float* decay_head,
                                     const float* a, const float* b, const float* denom_floor, float denom_eps,
                                     float* denom, float* state, int head_stride, int normaliser, const int* slots,
                                     const int* cu_q, int rows, int N, int H, int D, int V, float* out,
                                     cudaStream_t stream) {
    if (rows <= 0 || N <= 0) return EMS_OK;
    if (H <= 0 || D <= 0 || V <= 0 || (!decay_head && !a) || (normaliser && (!denom || !denom_floor)) ||
        head_stride < D * V + (normaliser ? D : 0) || H > 65535 || rows > 65535)
        return EMS_ERR_SHAPE;
    MatRecParams p;
    p.q = q; p.k = k; p.v = v; p.ldq = ldq; p.ldk = ldk; p.ldv = ldv; p.decay_head = decay_head; p.a = a; p.b = b;
    p.denom_floor = denom_floor; p.denom = denom; p.state = state; p.slots = slots; p.cu_q = cu_q; p.out = out;
    p.H = H; p.D = D; p.V = V; p.head_stride = head_stride; p.normaliser = normaliser; p.act = act;
    p.q_scale = q_scale; p.denom_eps = denom_eps;
    if (dtype == EMS_F32) return launch_matrix_recurrence<float>(p, rows, stream);
    if (dtype == EMS_BF16) return launch_matrix_recurrence<bf16>(p, rows, stream);
    return EMS_ERR_DTYPE;
}

EMS_EXPORT int ems_mlstm_gates(const float* pre, const void* bias_i, const void* bias_f, int b_dtype, float cap,
                               float* state, int head_stride, int m_offset, const int* slots, const int* cu_q,
                               int rows, int H, float* a_out, float* b_out, float* floor_out, cudaStream_t stream) {
    if (rows <= 0) return EMS_OK;
    if (H <= 0 || m_offset < 0 || m_offset >= head_stride) return EMS_ERR_SHAPE;
    const int warps = 4;
    mlstm_gates_kernel<<<(rows * H + warps - 1) / warps, warps * 32, 0, stream>>>(
        pre, bias_i, bias_f, b_dtype, cap, state, head_stride, m_offset, slots, cu_q, rows, H, a_out, b_out, floor_out);
    return launch_status();
}

EMS_EXPORT int ems_group_norm_gate(const float* o, const float* denom, const void* w, int w_dtype, const void* gate,
                                   long long ldg, void* out, int dtype, int N, int C, int groups, float eps,
                                   cudaStream_t stream) {
    if (N <= 0) return EMS_OK;
    if (groups <= 0 || C % groups) return EMS_ERR_SHAPE;
    const int gs = C / groups;
    const long long units = (long long)N * groups;
#define EMS_LAUNCH_GNG(T)                                                                                        \
    do {                                                                                                         \
        if (gs > 256)                                                                                            \
            group_norm_gate_kernel<T, true><<<(unsigned)units, gs > 1024 ? 256 : 128, 0, stream>>>(              \
                o, denom, w, w_dtype, (const T*)gate, ldg, (T*)out, N, C, groups, eps);                          \
        else                                                                                                     \
            group_norm_gate_kernel<T, false><<<(unsigned)((units + 3) / 4), 128, 0, stream>>>(                   \
                o, denom, w, w_dtype, (const T*)gate, ldg, (T*)out, N, C, groups, eps);                          \
    } while (0)
    if (dtype == EMS_F32) EMS_LAUNCH_GNG(float);
    else if (dtype == EMS_BF16) EMS_LAUNCH_GNG(bf16);
    else return EMS_ERR_DTYPE;
#undef EMS_LAUNCH_GNG
    return launch_status();
}

EMS_EXPORT int ems_rglru_scan(const void* u, const float* pre, const void* br, const void* bi, const void* lam,
                              int p_dtype, const void* y, long long ldy, int y_act, float cmul, float* state,
                              const int* slots, const int* cu_q, void* out, int dtype, int rows, int N, int C,
                              int blocks, cudaStream_t stream) {
    if (rows <= 0 || N <= 0) return EMS_OK;
    if (blocks <= 0 || C % blocks || rows > 65535) return EMS_ERR_SHAPE;
    const int th = C >= 128 ? 128 : 32 * ((C + 31) / 32);
    const dim3 grid((C + th - 1) / th, rows);
    if (dtype == EMS_F32)
        rglru_scan_kernel<float><<<grid, th, 0, stream>>>((const float*)u, pre, br, bi, lam, p_dtype, (const float*)y,
                                                          ldy, y_act, cmul, state, slots, cu_q, (float*)out, N, C,
                                                          blocks);
    else if (dtype == EMS_BF16)
        rglru_scan_kernel<bf16><<<grid, th, 0, stream>>>((const bf16*)u, pre, br, bi, lam, p_dtype, (const bf16*)y,
                                                         ldy, y_act, cmul, state, slots, cu_q, (bf16*)out, N, C,
                                                         blocks);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}
