// Routed experts: a router that scores all experts per token, the choice of the `top` best, and
// the experts' gated feed-forwards run as two grouped matrix products over the (token, choice)
// pairs sorted by expert.
//
//   route     z[t, :] are the router's logits (32-bit, computed by the caller);
//             s = softmax(z) over all experts; the `top` largest (ties: the lower index) are
//             chosen; their weights are the scores s as they are (renorm = 0) or divided by
//             their sum (renorm = 1).  The same kernel counts the pairs per expert, lays the
//             pairs out expert by expert (perm) and cuts each expert's rows into tiles.
//   up        act[i, :] = f(x[token(i)] Wg[e]^T) * (x[token(i)] Wu[e]^T)   for sorted pair i of expert e
//   down      y[pair(i), :] = act[i, :] Wd[e]^T            (32-bit, in pair order)
//   combine   out[t, :] = sum_k weight[t, k] * y[t * top + k, :]   (k ascending: a fixed order)
//
// A row of a product is computed by one thread column over K in ascending order, whatever else
// is in its tile: a token's result does not depend on the batch.  Products accumulate in 32 bits
// on the CUDA cores for both storage types.
#include "common.cuh"

namespace ems {

constexpr int MOE_TM = 64, MOE_TN = 64, MOE_TK = 16;

// plan (int32): [0] number of tiles; [1 .. 1 + 3 * max_tiles) expert, first sorted row and row
// count of each tile.  One block.
__global__ void moe_route_kernel(const float* __restrict__ logits, int n, int E, int top, int renorm,
                                 int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ offsets,
                                 int* __restrict__ perm, int* __restrict__ plan, int max_tiles) {
    extern __shared__ int sh[];
    int* counts = sh;       // [E]
    int* cursor = sh + E;   // [E]
    int* offs = sh + 2 * E; // [E + 1]
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int t = threadIdx.x; t < n; t += blockDim.x) {
        const float* z = logits + (size_t)t * E;
        float mx = -INFINITY;
        for (int e = 0; e < E; ++e) mx = fmaxf(mx, z[e]);
        float sum = 0.f;
        for (int e = 0; e < E; ++e) sum += expf(z[e] - mx);
        float chosen_sum = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < E; ++e) {
                bool taken = false;
                for (int j = 0; j < k; ++j) taken |= ids[(size_t)t * top + j] == e;
                if (!taken && (best < 0 || z[e] > bv)) {
                    best = e;
                    bv = z[e];
                }
            }
            ids[(size_t)t * top + k] = best;
            const float s = expf(bv - mx) / sum;
            wts[(size_t)t * top + k] = s;
            chosen_sum += s;
            atomicAdd(&counts[best], 1);
        }
        if (renorm)
            for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] /= chosen_sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            offs[e] = run;
            offsets[e] = run;
            cursor[e] = 0;
            for (int r0 = 0; r0 < counts[e] && nt < max_tiles; r0 += MOE_TM, ++nt) {
                plan[1 + 3 * nt] = e;
                plan[2 + 3 * nt] = run + r0;
                plan[3 + 3 * nt] = min(MOE_TM, counts[e] - r0);
            }
            run += counts[e];
        }
        offs[E] = run;
        offsets[E] = run;
        plan[0] = nt;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < n; t += blockDim.x)
        for (int k = 0; k < top; ++k) {
            const int e = ids[(size_t)t * top + k];
            perm[offs[e] + atomicAdd(&cursor[e], 1)] = t * top + k;
        }
}

__device__ __forceinline__ float moe_activation(float g, int act) {
    if (act == 1) return fmaxf(g, 0.f);
    if (act == 2) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.f + expf(-g));
}

// GLU = true:  A rows are x[perm[row] / top] (gathered), B = w[e] of shape [2 N, K]; the tile
//              computes gate and up columns side by side and stores f(gate) * up in sorted order.
// GLU = false: A rows are a[row] (sorted order), B = w[e] of shape [N, K]; the tile is stored at
//              rows perm[row] of a 32-bit output.
template <typename T, bool GLU>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const T* __restrict__ a, const T* __restrict__ w, const int* __restrict__ perm,
                   const int* __restrict__ plan, int top, int N, int K, int act, T* __restrict__ out_t,
                   float* __restrict__ out_f) {
    __shared__ float As[MOE_TK][MOE_TM + 4];
    __shared__ float Bs[MOE_TK][MOE_TN + 4];
    __shared__ float Bu[GLU ? MOE_TK : 1][MOE_TN + 4];
    __shared__ int src_row[MOE_TM];
    const int tile = blockIdx.x;
    if (tile >= plan[0]) return;
    const int e = plan[1 + 3 * tile], row0 = plan[2 + 3 * tile], rows = plan[3 + 3 * tile];
    const int n0 = blockIdx.y * MOE_TN;
    const T* we = w + (size_t)e * (GLU ? 2 : 1) * N * K;
    for (int i = threadIdx.x; i < MOE_TM; i += blockDim.x)
        src_row[i] = i < rows ? (GLU ? perm[row0 + i] / top : row0 + i) : -1;
    __syncthreads();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int lr = threadIdx.x / 4, lk = (threadIdx.x % 4) * 4;  // the loader's row and first column
    float cg[4][4], cu[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) cg[i][j] = cu[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MOE_TK) {
        const int ar = src_row[lr];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            As[lk + j][lr] = (ar >= 0 && k < K) ? to_f32<T>(a[(size_t)ar * K + k]) : 0.f;
            const int nn = n0 + lr;
            const bool ok = nn < N && k < K;
            Bs[lk + j][lr] = ok ? to_f32<T>(we[(size_t)nn * K + k]) : 0.f;
            if (GLU) Bu[lk + j][lr] = ok ? to_f32<T>(we[(size_t)(N + nn) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_TK; ++kk) {
            float av[4], bv[4], uv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                bv[j] = Bs[kk][tx * 4 + j];
                if (GLU) uv[j] = Bu[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    cg[i][j] = fmaf(av[i], bv[j], cg[i][j]);
                    if (GLU) cu[i][j] = fmaf(av[i], uv[j], cu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx * 4 + j;
            if (c >= N) continue;
            if (GLU) {
                // both projections are rounded to the storage type before the activation, as a
                // product that is stored and read again would be
                const float g = round_to<T>(cg[i][j]), u = round_to<T>(cu[i][j]);
                out_t[(size_t)(row0 + r) * N + c] = from_f32<T>(moe_activation(g, act) * u);
            } else {
                out_f[(size_t)perm[row0 + r] * N + c] = round_to<T>(cg[i][j]);
            }
        }
    }
}

template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ wts, T* __restrict__ out,
                                   int top, int H) {
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) s = fmaf(wts[t * top + k], y[(t * top + k) * H + c], s);
        out[t * H + c] = from_f32<T>(s);
    }
}

}  // namespace ems

using namespace ems;

EMS_EXPORT int ems_moe_tile_rows() { return MOE_TM; }

EMS_EXPORT int ems_moe_route(const float* logits, int n, int E, int top, int renorm, int* ids, float* wts,
                             int* offsets, int* perm, int* plan, int max_tiles, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (top < 1 || top > E) return EMS_ERR_SHAPE;
    const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
    if (smem > 48 * 1024) return EMS_ERR_SHAPE;
    int th = 32;
    while (th < n && th < 1024) th <<= 1;
    moe_route_kernel<<<1, th, smem, stream>>>(logits, n, E, top, renorm, ids, wts, offsets, perm, plan, max_tiles);
    return launch_status();
}

EMS_EXPORT int ems_moe_up(const void* x, const void* wgu, int dtype, const int* perm, const int* plan, int max_tiles,
                          int top, int ff, int K, int act, void* out, cudaStream_t stream) {
    if (max_tiles <= 0) return EMS_OK;
    dim3 grid(max_tiles, (ff + MOE_TN - 1) / MOE_TN);
    if (dtype == EMS_F32)
        moe_grouped_kernel<float, true><<<grid, 256, 0, stream>>>((const float*)x, (const float*)wgu, perm, plan, top,
                                                                  ff, K, act, (float*)out, nullptr);
    else if (dtype == EMS_BF16)
        moe_grouped_kernel<bf16, true><<<grid, 256, 0, stream>>>((const bf16*)x, (const bf16*)wgu, perm, plan, top,
                                                                 ff, K, act, (bf16*)out, nullptr);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_moe_down(const void* a, const void* wdown, int dtype, const int* perm, const int* plan,
                            int max_tiles, int H, int ff, float* y, cudaStream_t stream) {
    if (max_tiles <= 0) return EMS_OK;
    dim3 grid(max_tiles, (H + MOE_TN - 1) / MOE_TN);
    if (dtype == EMS_F32)
        moe_grouped_kernel<float, false><<<grid, 256, 0, stream>>>((const float*)a, (const float*)wdown, perm, plan, 1,
                                                                   H, ff, 0, nullptr, y);
    else if (dtype == EMS_BF16)
        moe_grouped_kernel<bf16, false><<<grid, 256, 0, stream>>>((const bf16*)a, (const bf16*)wdown, perm, plan, 1,
                                                                  H, ff, 0, nullptr, y);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_moe_combine(const float* y, const float* wts, void* out, int dtype, int n, int top, int H,
                               cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    int th = 32;
    while (th < H && th < 256) th <<= 1;
    if (dtype == EMS_F32) moe_combine_kernel<float><<<n, th, 0, stream>>>(y, wts, (float*)out, top, H);
    else if (dtype == EMS_BF16) moe_combine_kernel<bf16><<<n, th, 0, stream>>>(y, wts, (bf16*)out, top, H);
    else return EMS_ERR_DTYPE;
    return launch_status();
}
