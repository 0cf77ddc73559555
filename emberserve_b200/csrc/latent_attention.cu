// Latent attention: every token keeps ONE vector of R + P numbers in the paged cache, the
// normed latent c (R numbers) and a rotated key part shared by all heads (P numbers).  Keys and
// values of a head are linear maps of c, so the attention runs on the latent itself:
//
//   score(i, j, h) = (qlat[h, i, :] . c[j, :] + qrot[i, h, :] . krot[j, :]) * scale
//   olat[h, i, :]  = sum_j softmax_j(score(i, :, h)) * c[j, :]
//
// with qlat[h] = q_plain[h] Wuk[h] (the key up-projection folded into the query) and the value
// up-projection applied to olat afterwards; both are batched matrix products outside this file.
// All heads read the same R + P numbers per key, which is why one block serves several heads.
//
// Kernels: the preparation of a step's tokens (the two RMSNorms of the down-projections, the
// rotation of the shared key part, the cache write), a rotation in place for the query heads, the
// attention itself with an optional split of the keys over several blocks, the merge of such
// splits, and the output gate with the transposition back to token-major rows.
// Scores, softmax and the weighted sums are 32-bit; T is the storage type (float or bfloat16).
// In bfloat16 the attention runs on the tensor cores where the sizes allow (latent_attention_mma.cu);
// the kernel here serves the 32-bit path and every other geometry.
#include "latent_attention.cuh"

namespace ems {

// Rotation of `dims` leading numbers of a vector: pairing 0 joins entry i with i + dims/2,
// pairing 1 joins entry 2i with 2i + 1.  table: [pos, dims/2, 2] (cos, sin).
__device__ __forceinline__ void pair_index(int i, int dims, int pairing, int& a, int& b) {
    if (pairing == 0) { a = i; b = i + dims / 2; }
    else { a = 2 * i; b = 2 * i + 1; }
}

// ---------------------------------------------------------------------------------------
// One block per token.  proj row: [q latent (QR) | kv latent (R) | shared key part (P) | ...].

template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, int proj_stride, int QR, int R, int P,
                                   const void* __restrict__ q_gain, const void* __restrict__ kv_gain, int g_dtype,
                                   float eps, const int* __restrict__ positions,
                                   const int* __restrict__ row_of_token, const float* __restrict__ table,
                                   int rot_dims, int pairing, T* __restrict__ pages,
                                   const int* __restrict__ block_tables, int bt_stride, int page_size,
                                   T* __restrict__ cq, int write) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const T* p = proj + (size_t)t * proj_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < QR; i += blockDim.x) {
        const float v = to_f32<T>(p[i]);
        ss += v * v;
    }
    const float q_rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)QR + eps);
    for (int i = threadIdx.x; i < QR; i += blockDim.x)
        cq[(size_t)t * QR + i] = from_f32<T>(to_f32<T>(p[i]) * q_rstd * load_any(q_gain, g_dtype, i));
    if (!write) return;
    ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = to_f32<T>(p[QR + i]);
        ss += v * v;
    }
    const float kv_rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)R + eps);
    const int pos = positions[t];
    const int page = block_tables[(size_t)row_of_token[t] * bt_stride + pos / page_size];
    T* dst = pages + ((size_t)page * page_size + pos % page_size) * (R + P);
    for (int i = threadIdx.x; i < R; i += blockDim.x)
        dst[i] = from_f32<T>(to_f32<T>(p[QR + i]) * kv_rstd * load_any(kv_gain, g_dtype, i));
    const T* kr = p + QR + R;
    const float* cs = table + (size_t)pos * (rot_dims / 2) * 2;
    for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
        int a, b;
        pair_index(i, rot_dims, pairing, a, b);
        const float u = to_f32<T>(kr[a]), v = to_f32<T>(kr[b]), c = cs[2 * i], s = cs[2 * i + 1];
        dst[R + a] = from_f32<T>(u * c - v * s);
        dst[R + b] = from_f32<T>(v * c + u * s);
    }
    for (int i = rot_dims + threadIdx.x; i < P; i += blockDim.x) dst[R + i] = kr[i];
}

// x[t, h, offset + ...] rotated in place; x row stride and head stride in elements.
template <typename T>
__global__ void rope_inplace_kernel(T* __restrict__ x, int row_stride, int head_stride, int offset, int heads,
                                    int rot_dims, int pairing, const int* __restrict__ positions,
                                    const float* __restrict__ table) {
    const int t = blockIdx.x;
    const int half = rot_dims / 2;
    const float* cs = table + (size_t)positions[t] * half * 2;
    for (int k = threadIdx.x; k < heads * half; k += blockDim.x) {
        const int h = k / half, i = k % half;
        int a, b;
        pair_index(i, rot_dims, pairing, a, b);
        T* v = x + (size_t)t * row_stride + (size_t)h * head_stride + offset;
        const float u = to_f32<T>(v[a]), w = to_f32<T>(v[b]), c = cs[2 * i], s = cs[2 * i + 1];
        v[a] = from_f32<T>(u * c - w * s);
        v[b] = from_f32<T>(w * c + u * s);
    }
}

// ---------------------------------------------------------------------------------------
// The attention.  Block (token, split, head chunk); its warps take turns over tiles of 32 keys.
// In a tile a lane owns one key for the scores (all HC heads of the chunk) and, for the weighted
// sum, the latent entries lane, lane + 32, ... (NR of them) of every key.

constexpr int LA_TILE = 32;

template <typename T> struct Word;  // 4 bytes of T as floats
template <> struct Word<float> {
    static constexpr int N = 1;
    static __device__ __forceinline__ void get(const uint32_t w, float (&v)[2]) { v[0] = __uint_as_float(w); v[1] = 0.f; }
};
template <> struct Word<bf16> {
    static constexpr int N = 2;
    static __device__ __forceinline__ void get(const uint32_t w, float (&v)[2]) {
        v[0] = __uint_as_float(w << 16);
        v[1] = __uint_as_float(w & 0xffff0000u);
    }
};

template <typename T, int HC, int NR>
__global__ void latent_attention_kernel(const T* __restrict__ qlat, const T* __restrict__ qrot, int q_row_stride,
                                        int q_head_stride, const T* __restrict__ pages,
                                        const int* __restrict__ block_tables, int bt_stride, int page_size,
                                        const int* __restrict__ positions, const int* __restrict__ row_of_token,
                                        T* __restrict__ out, float* __restrict__ partial, int num_tokens, int H,
                                        int R, int P, int DPW, float scale, int splits) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int EPW = Word<T>::N;
    const int D = R + P;
    const int W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x, sp = blockIdx.y, h0 = blockIdx.z * HC;
    float* q_s = reinterpret_cast<float*>(smem_raw);                       // [HC][D]
    float* p_s = q_s + HC * D + warp * HC * LA_TILE;                       // [W][HC][32]
    float* ml_s = q_s + HC * D + W * HC * LA_TILE;                         // [W][HC][2]
    uint32_t* tiles = reinterpret_cast<uint32_t*>(ml_s + W * HC * 2);      // [W][32][DPW] words
    uint32_t* ktile = tiles + (size_t)warp * LA_TILE * DPW;
    float* acc_s = reinterpret_cast<float*>(tiles);                        // [W][HC][R], after the key loop

    for (int k = threadIdx.x; k < HC * D; k += blockDim.x) {
        const int h = k / D, d = k % D;
        float v = 0.f;
        if (h0 + h < H)
            v = d < R ? to_f32<T>(qlat[((size_t)(h0 + h) * num_tokens + t) * R + d])
                      : to_f32<T>(qrot[(size_t)t * q_row_stride + (size_t)(h0 + h) * q_head_stride + (d - R)]);
        q_s[k] = v;
    }
    __syncthreads();

    const int qpos = positions[t];
    const int* bt = block_tables + (size_t)row_of_token[t] * bt_stride;
    const int kend = qpos + 1;  // causal: keys 0 .. qpos
    int chunk = (kend + splits - 1) / splits;
    chunk = (chunk + LA_TILE - 1) / LA_TILE * LA_TILE;
    const int k_lo = sp * chunk, k_hi = min(kend, k_lo + chunk);

    float m[HC], l[HC], acc[HC][NR];
#pragma unroll
    for (int h = 0; h < HC; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.f;
#pragma unroll
        for (int i = 0; i < NR; ++i) acc[h][i] = 0.f;
    }
    const int row_words = D / EPW;  // words of a cached vector

    for (int k0 = k_lo + warp * LA_TILE; k0 < k_hi; k0 += W * LA_TILE) {
        // stage the tile: key k0 + j into row j (zeros past the last visible key)
        const int mykey = k0 + lane;
        const uint32_t* myrow = nullptr;
        if (mykey < k_hi)
            myrow = reinterpret_cast<const uint32_t*>(
                pages + ((size_t)bt[mykey / page_size] * page_size + mykey % page_size) * D);
        for (int j = 0; j < LA_TILE; ++j) {
            const uint32_t* src = reinterpret_cast<const uint32_t*>(
                __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(myrow), j));
            for (int w = lane; w < row_words; w += 32) ktile[j * DPW + w] = src ? src[w] : 0u;
        }
        __syncwarp();
        // scores of my key
        float s[HC];
#pragma unroll
        for (int h = 0; h < HC; ++h) s[h] = 0.f;
        const uint32_t* kr = ktile + lane * DPW;
        for (int w = 0; w < row_words; ++w) {
            float kv[2];
            Word<T>::get(kr[w], kv);
#pragma unroll
            for (int e = 0; e < EPW; ++e) {
#pragma unroll
                for (int h = 0; h < HC; ++h) s[h] = fmaf(q_s[h * D + w * EPW + e], kv[e], s[h]);
            }
        }
        const bool valid = mykey < k_hi;
#pragma unroll
        for (int h = 0; h < HC; ++h) {
            const float sc = valid ? s[h] * scale : -INFINITY;
            const float m_new = fmaxf(m[h], warp_max(sc));
            const float alpha = expf(m[h] - m_new);  // 0 at the first tile (m = -inf, m_new finite)
            const float p = valid ? expf(sc - m_new) : 0.f;
            l[h] = l[h] * alpha + p;
            m[h] = m_new;
            p_s[h * LA_TILE + lane] = p;
#pragma unroll
            for (int i = 0; i < NR; ++i) acc[h][i] *= alpha;
        }
        __syncwarp();
        const int nkeys = min(LA_TILE, k_hi - k0);
        const T* kt = reinterpret_cast<const T*>(ktile);
        for (int j = 0; j < nkeys; ++j) {
            float c[NR];
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                const int r = lane + 32 * i;
                c[i] = r < R ? to_f32<T>(kt[(size_t)j * DPW * EPW + r]) : 0.f;
            }
#pragma unroll
            for (int h = 0; h < HC; ++h) {
                const float p = p_s[h * LA_TILE + j];
#pragma unroll
                for (int i = 0; i < NR; ++i) acc[h][i] = fmaf(p, c[i], acc[h][i]);
            }
        }
        __syncwarp();
    }
    // merge the warps
    __syncthreads();
#pragma unroll
    for (int h = 0; h < HC; ++h) {
        const float lt = warp_sum(l[h]);
        if (lane == 0) {
            ml_s[(warp * HC + h) * 2] = m[h];
            ml_s[(warp * HC + h) * 2 + 1] = lt;
        }
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int r = lane + 32 * i;
            if (r < R) acc_s[((size_t)warp * HC + h) * R + r] = acc[h][i];
        }
    }
    __syncthreads();
    for (int k = threadIdx.x; k < HC * R; k += blockDim.x) {
        const int h = k / R, r = k % R;
        if (h0 + h >= H) continue;
        float M = -INFINITY;
        for (int w = 0; w < W; ++w) M = fmaxf(M, ml_s[(w * HC + h) * 2]);
        float L = 0.f, O = 0.f;
        if (M > -INFINITY) {
            for (int w = 0; w < W; ++w) {
                const float f = expf(ml_s[(w * HC + h) * 2] - M);
                L += ml_s[(w * HC + h) * 2 + 1] * f;
                O += acc_s[((size_t)w * HC + h) * R + r] * f;
            }
        }
        if (splits == 1) {
            out[((size_t)(h0 + h) * num_tokens + t) * R + r] = from_f32<T>(O / L);
        } else {
            float* dst = partial + (((size_t)t * H + (h0 + h)) * splits + sp) * (R + 2);
            dst[r] = O;
            if (r == 0) {
                dst[R] = M;
                dst[R + 1] = L;
            }
        }
    }
}

// partial: [token, head, split, R + 2] (unnormalised sums, then running maximum and sum).
template <typename T>
__global__ void latent_attention_merge_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                              int num_tokens, int H, int R, int splits) {
    const int t = blockIdx.x, h = blockIdx.y;
    const float* src = partial + ((size_t)t * H + h) * splits * (R + 2);
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, src[(size_t)s * (R + 2) + R]);
    float L = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = src[(size_t)s * (R + 2) + R];
        if (ms > -INFINITY) L += src[(size_t)s * (R + 2) + R + 1] * expf(ms - M);
    }
    for (int r = threadIdx.x; r < R; r += blockDim.x) {
        float O = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = src[(size_t)s * (R + 2) + R];
            if (ms > -INFINITY) O += src[(size_t)s * (R + 2) + r] * expf(ms - M);
        }
        out[((size_t)h * num_tokens + t) * R + r] = from_f32<T>(O / L);
    }
}

// out[t, h * V + i] = ov[h, t, i] * sigmoid(gate[t, h * V + i])   (no gate: a plain transposition)
template <typename T>
__global__ void heads_gate_kernel(const T* __restrict__ ov, const T* __restrict__ gate, int gate_stride,
                                  T* __restrict__ out, int num_tokens, int H, int V) {
    const int t = blockIdx.x;
    for (int k = threadIdx.x; k < H * V; k += blockDim.x) {
        const int h = k / V, i = k % V;
        float v = to_f32<T>(ov[((size_t)h * num_tokens + t) * V + i]);
        if (gate) {
            const float g = to_f32<T>(gate[(size_t)t * gate_stride + k]);
            v = v / (1.f + expf(-g));
        }
        out[(size_t)t * H * V + k] = from_f32<T>(v);
    }
}

static int la_threads_for(int n) {
    int t = 32;
    while (t < n && t < 256) t <<= 1;
    return t;
}

// Words per staged key row: the row's own words rounded up to an odd count, so that the 32 lanes
// of a warp, each walking along its own row, hit 32 different banks.
static int la_row_words(int D, int esize) {
    const int words = D * esize / 4;
    return words | 1;
}

template <typename T, int HC, int NR>
static int launch_latent_attention(const void* qlat, const void* qrot, int q_row_stride, int q_head_stride,
                                   const void* pages, const int* block_tables, int bt_stride, int page_size,
                                   const int* positions, const int* row_of_token, void* out, float* partial,
                                   int num_tokens, int H, int R, int P, float scale, int splits, cudaStream_t stream) {
    const int D = R + P;
    const int dpw = la_row_words(D, (int)sizeof(T));
    int warps = 4;
    size_t smem = 0;
    for (; warps >= 1; warps >>= 1) {
        smem = (size_t)HC * D * 4 + (size_t)warps * HC * LA_TILE * 4 + (size_t)warps * HC * 2 * 4 +
               (size_t)warps * LA_TILE * dpw * 4;
        if (smem <= 200 * 1024) break;
    }
    if (warps < 1) return EMS_ERR_SHAPE;
    auto kern = latent_attention_kernel<T, HC, NR>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return EMS_ERR_LAUNCH;
    }
    dim3 grid(num_tokens, splits, (H + HC - 1) / HC);
    kern<<<grid, warps * 32, smem, stream>>>((const T*)qlat, (const T*)qrot, q_row_stride, q_head_stride,
                                             (const T*)pages, block_tables, bt_stride, page_size, positions,
                                             row_of_token, (T*)out, partial, num_tokens, H, R, P, dpw, scale, splits);
    if (splits > 1) {
        dim3 mg(num_tokens, H);
        latent_attention_merge_kernel<T><<<mg, la_threads_for(R), 0, stream>>>(partial, (T*)out, num_tokens, H, R,
                                                                               splits);
    }
    return launch_status();
}

template <typename T>
static int dispatch_latent_attention(const void* qlat, const void* qrot, int q_row_stride, int q_head_stride,
                                     const void* pages, const int* block_tables, int bt_stride, int page_size,
                                     const int* positions, const int* row_of_token, void* out, float* partial,
                                     int num_tokens, int H, int R, int P, float scale, int splits,
                                     cudaStream_t stream) {
#define EMS_LA(HC, NR)                                                                                            \
    return launch_latent_attention<T, HC, NR>(qlat, qrot, q_row_stride, q_head_stride, pages, block_tables,       \
                                              bt_stride, page_size, positions, row_of_token, out, partial,        \
                                              num_tokens, H, R, P, scale, splits, stream)
    if (R <= 128) EMS_LA(8, 4);
    if (R <= 256) EMS_LA(8, 8);
    if (R <= 512) EMS_LA(4, 16);
#undef EMS_LA
    return EMS_ERR_SHAPE;
}

}  // namespace ems

using namespace ems;

EMS_EXPORT int ems_latent_prep(const void* proj, int proj_stride, int dtype, int n, int QR, int R, int P,
                               const void* q_gain, const void* kv_gain, int g_dtype, float eps,
                               const int* positions, const int* row_of_token, const float* table, int rot_dims,
                               int pairing, void* pages, const int* block_tables, int bt_stride, int page_size,
                               void* cq, int write, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > P || (rot_dims > 0 && !table)) return EMS_ERR_SHAPE;
    const int th = la_threads_for(QR > R ? QR : R);
    if (dtype == EMS_F32)
        latent_prep_kernel<float><<<n, th, 0, stream>>>((const float*)proj, proj_stride, QR, R, P, q_gain, kv_gain,
                                                        g_dtype, eps, positions, row_of_token, table, rot_dims,
                                                        pairing, (float*)pages, block_tables, bt_stride, page_size,
                                                        (float*)cq, write);
    else if (dtype == EMS_BF16)
        latent_prep_kernel<bf16><<<n, th, 0, stream>>>((const bf16*)proj, proj_stride, QR, R, P, q_gain, kv_gain,
                                                       g_dtype, eps, positions, row_of_token, table, rot_dims,
                                                       pairing, (bf16*)pages, block_tables, bt_stride, page_size,
                                                       (bf16*)cq, write);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_rope_inplace(void* x, int dtype, int n, int row_stride, int head_stride, int offset, int heads,
                                int rot_dims, int pairing, const int* positions, const float* table,
                                cudaStream_t stream) {
    if (n <= 0 || rot_dims == 0) return EMS_OK;
    if (rot_dims % 2 || !table) return EMS_ERR_SHAPE;
    const int th = la_threads_for(heads * rot_dims / 2);
    if (dtype == EMS_F32)
        rope_inplace_kernel<float><<<n, th, 0, stream>>>((float*)x, row_stride, head_stride, offset, heads, rot_dims,
                                                         pairing, positions, table);
    else if (dtype == EMS_BF16)
        rope_inplace_kernel<bf16><<<n, th, 0, stream>>>((bf16*)x, row_stride, head_stride, offset, heads, rot_dims,
                                                        pairing, positions, table);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT long long ems_latent_attention_scratch_bytes(int num_tokens, int H, int R, int splits) {
    return splits <= 1 ? 0 : (long long)num_tokens * H * splits * (R + 2) * 4;
}

EMS_EXPORT int ems_latent_attention(const void* qlat, const void* qrot, int q_row_stride, int q_head_stride,
                                    int dtype, const void* pages, const int* block_tables, int bt_stride,
                                    int page_size, const int* positions, const int* row_of_token, void* out,
                                    int num_tokens, int H, int R, int P, float scale, int splits, void* scratch,
                                    long long scratch_bytes, int impl, cudaStream_t stream) {
    if (num_tokens <= 0) return EMS_OK;
    if (splits < 1 || splits > 65535) return EMS_ERR_SHAPE;
    if (dtype == EMS_BF16 && ((R + P) % 2)) return EMS_ERR_SHAPE;  // a cached vector is read in 4-byte words
    if (splits > 1 && (!scratch || scratch_bytes < ems_latent_attention_scratch_bytes(num_tokens, H, R, splits)))
        return EMS_ERR_SCRATCH;
    // impl: 0 the tensor-core kernel where it takes the case, 1 always the generic kernel
    if (dtype == EMS_BF16 && impl == 0 &&
        latent_mma_supported(R, P, qlat, qrot, q_row_stride, q_head_stride, pages)) {
        const int rc = run_latent_mma(qlat, qrot, q_row_stride, q_head_stride, pages, block_tables, bt_stride,
                                      page_size, positions, row_of_token, out, (float*)scratch, num_tokens, H, R, P,
                                      scale, splits, stream);
        if (rc != EMS_OK || splits == 1) return rc;
        dim3 mg(num_tokens, H);
        latent_attention_merge_kernel<bf16><<<mg, la_threads_for(R), 0, stream>>>((const float*)scratch, (bf16*)out,
                                                                                  num_tokens, H, R, splits);
        return launch_status();
    }
    if (dtype == EMS_F32)
        return dispatch_latent_attention<float>(qlat, qrot, q_row_stride, q_head_stride, pages, block_tables,
                                                bt_stride, page_size, positions, row_of_token, out, (float*)scratch,
                                                num_tokens, H, R, P, scale, splits, stream);
    if (dtype == EMS_BF16)
        return dispatch_latent_attention<bf16>(qlat, qrot, q_row_stride, q_head_stride, pages, block_tables,
                                               bt_stride, page_size, positions, row_of_token, out, (float*)scratch,
                                               num_tokens, H, R, P, scale, splits, stream);
    return EMS_ERR_DTYPE;
}

EMS_EXPORT int ems_heads_gate(const void* ov, const void* gate, int gate_stride, void* out, int dtype, int n, int H,
                              int V, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    const int th = la_threads_for(H * V);
    if (dtype == EMS_F32)
        heads_gate_kernel<float><<<n, th, 0, stream>>>((const float*)ov, (const float*)gate, gate_stride,
                                                       (float*)out, n, H, V);
    else if (dtype == EMS_BF16)
        heads_gate_kernel<bf16><<<n, th, 0, stream>>>((const bf16*)ov, (const bf16*)gate, gate_stride, (bf16*)out,
                                                      n, H, V);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}
