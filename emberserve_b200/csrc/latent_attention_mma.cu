// Latent attention on the tensor cores (bfloat16): the same computation as the generic kernel of
// latent_attention.cu, as two mma.sync m16n8k16 products per tile of keys.
//
// A block serves ONE token and up to 16 of its heads: the heads are the 16 rows of the m16 tile,
// and all of them read the same cached vectors [c | krot] (R + P numbers per key), so a tile of
// 64 keys in shared memory feeds both products:
//   S[16, 64]  = Q[16, R + P] K^T          K rows as they lie in the cache (ldmatrix)
//   O[16, R]  += P[16, 64] K[:, :R]        the same rows, read transposed (ldmatrix.trans)
// The warps (four, or eight for long latents) share the keys of a tile for the scores and the latent
// columns of O for the second product.  Scores, running maximum and sums are float32; the weights are
// rounded to bfloat16 for the second product.  Tiles arrive by cp.async (a two-stage ring where two
// blocks with two stages each fit an SM, one stage otherwise);
// rows past the last visible key are filled with zeros.  With `splits` > 1 a block takes a range
// of the keys and leaves unnormalised sums, maximum and sum for the merge kernel.
#include "latent_attention.cuh"

namespace ems {

constexpr int LM_KT = 64;     // keys per tile
constexpr int LM_PAD = 8;     // bfloat16 of padding per shared-memory row

__device__ __forceinline__ void lm_cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void lm_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void lm_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void lm_ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_ldmatrix_x2_trans(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void lm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// W warps per block (4 or 8); NTW: the most 8-column tiles of O a warp may own (R <= 8 * W * NTW).
// Warp w computes the scores of keys (64 / W) w .. of the tile and owns the latent columns
// [w R / W, (w + 1) R / W) of O.
template <int NTW, int W>
__global__ void __launch_bounds__(W * 32)
latent_attention_mma_kernel(const bf16* __restrict__ qlat, const bf16* __restrict__ qrot, int q_row_stride,
                            int q_head_stride, const bf16* __restrict__ pages, const int* __restrict__ block_tables,
                            int bt_stride, int page_size, const int* __restrict__ positions,
                            const int* __restrict__ row_of_token, bf16* __restrict__ out, float* __restrict__ partial,
                            int num_tokens, int H, int R, int P, float scale_log2, int splits, int stages) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    constexpr int KW = LM_KT / W;  // keys of a tile per warp: 16 or 8
    constexpr int NJ = KW / 8;     // 8-key tiles of the score product per warp
    const int D = R + P, DS = D + LM_PAD;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int t = blockIdx.x, sp = blockIdx.y, h0 = blockIdx.z * 16;
    bf16* Qs = reinterpret_cast<bf16*>(lm_smem);                  // [16][DS]
    bf16* Ks = Qs + 16 * DS;                                      // [stages][LM_KT][DS]
    bf16* Ps = Ks + stages * LM_KT * DS;                          // [16][LM_KT + LM_PAD]
    float* smax = reinterpret_cast<float*>(Ps + 16 * (LM_KT + LM_PAD));  // [W][16]
    float* ssum = smax + W * 16;                                  // [W][16]
    constexpr int PS = LM_KT + LM_PAD;

    const int qpos = positions[t];
    const int* bt = block_tables + (size_t)row_of_token[t] * bt_stride;
    const int kend = qpos + 1;
    int chunk = (kend + splits - 1) / splits;
    chunk = (chunk + LM_KT - 1) / LM_KT * LM_KT;
    const int k_lo = sp * chunk, k_hi = min(kend, k_lo + chunk);
    const int ntw = R / (8 * W);      // 8-column tiles of O per warp
    const int col0 = warp * (R / W);  // my first latent column

    float o[NTW][4];
#pragma unroll
    for (int i = 0; i < NTW; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // rows g and g + 8

    if (k_lo < k_hi) {
        // the queries: row = head, [folded query (R) | rotated part (P)]; the warps take heads in turn
        for (int row = warp; row < 16; row += W) {
            const bool live = h0 + row < H;
            const bf16* ql = qlat + ((size_t)(h0 + row) * num_tokens + t) * R;
            const bf16* qr = qrot + (size_t)t * q_row_stride + (size_t)(h0 + row) * q_head_stride;
            for (int d = 2 * lane; d < D; d += 64) {
                uint32_t v = 0u;
                if (live) v = *reinterpret_cast<const uint32_t*>(d < R ? ql + d : qr + (d - R));
                *reinterpret_cast<uint32_t*>(Qs + row * DS + d) = v;
            }
        }
        const int cpr = D / 8;  // 16-byte chunks per cached vector
        const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(Ks);
        // A warp copies the keys whose scores it will compute: lane r < KW finds the page slot of key
        // r (one look at the block table per key), the address goes round by shuffle, and the lanes
        // copy the vector 16 bytes each.
        auto prefetch = [&](int tile_k0, int stage) {
            const int mykey = tile_k0 + warp * KW + (lane & (KW - 1));
            const bf16* mine = nullptr;
            if (mykey < k_hi) mine = pages + ((size_t)bt[mykey / page_size] * page_size + mykey % page_size) * D;
#pragma unroll 4
            for (int r = 0; r < KW; ++r) {
                const bf16* src = reinterpret_cast<const bf16*>(
                    __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(mine), r));
                const bool valid = src != nullptr;
                const uint32_t dst = ks_base + (uint32_t)(((stage * LM_KT + warp * KW + r) * DS) * 2);
                for (int col = lane; col < cpr; col += 32)
                    lm_cp_async16(dst + col * 16, valid ? src + col * 8 : pages, valid);
            }
            lm_commit();
        };
        const uint32_t qs_addr = (uint32_t)__cvta_generic_to_shared(Qs);
        const uint32_t ps_addr = (uint32_t)__cvta_generic_to_shared(Ps);
        // ldmatrix addresses of this lane.  A tiles: row-major 16 x 16.  B tiles of the score product:
        // with 16 keys per warp, two key octets x the two halves of 16 columns; with 8 keys, one key
        // octet x four octets of 32 columns.  B tiles of the second product: transposed.
        const int a_row = (lane & 7) + 8 * ((lane >> 3) & 1), a_col = 8 * (lane >> 4);
        const int b_row = NJ == 2 ? (lane & 7) + 8 * (lane >> 4) : (lane & 7);
        const int b_col = NJ == 2 ? 8 * ((lane >> 3) & 1) : 8 * (lane >> 3);
        const int v_row = (lane & 7) + 8 * ((lane >> 3) & 1);

        // Two stages: the next tile travels while this one is used.  One stage (where two would leave
        // room for one block per SM only): a block waits for its tile, and the SM's other block computes.
        const int flip = stages - 1;
        if (flip) prefetch(k_lo, 0);
        int stage = 0;
        for (int k0 = k_lo; k0 < k_hi; k0 += LM_KT, stage ^= flip) {
            const bool more = k0 + LM_KT < k_hi;
            if (!flip) {
                prefetch(k0, 0);
                lm_wait<0>();
            } else if (more) {
                prefetch(k0 + LM_KT, stage ^ 1);
                lm_wait<1>();
            } else {
                lm_wait<0>();
            }
            __syncthreads();
            const uint32_t kst = ks_base + (uint32_t)(stage * LM_KT * DS * 2);
            // scores of my keys: two sets of sums over alternating slices of D keep more chains in flight
            float s[NJ][4], s2[NJ][4];
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
                s2[j][0] = s2[j][1] = s2[j][2] = s2[j][3] = 0.f;
            }
            const uint32_t qa = qs_addr + (uint32_t)((a_row * DS + a_col) * 2);
            const uint32_t kb = kst + (uint32_t)(((warp * KW + b_row) * DS + b_col) * 2);
            int kk = 0;
            for (; kk + 32 <= D; kk += 32) {
                uint32_t a[4], a2[4];
                lm_ldmatrix_x4(qa + kk * 2, a);
                lm_ldmatrix_x4(qa + (kk + 16) * 2, a2);
                if (NJ == 2) {
                    uint32_t b[4], b2[4];
                    lm_ldmatrix_x4(kb + kk * 2, b);
                    lm_ldmatrix_x4(kb + (kk + 16) * 2, b2);
                    lm_mma(s[0], a, b[0], b[1]);
                    lm_mma(s[NJ - 1], a, b[2], b[3]);
                    lm_mma(s2[0], a2, b2[0], b2[1]);
                    lm_mma(s2[NJ - 1], a2, b2[2], b2[3]);
                } else {
                    uint32_t b[4];  // one key octet, columns kk .. kk + 31
                    lm_ldmatrix_x4(kb + kk * 2, b);
                    lm_mma(s[0], a, b[0], b[1]);
                    lm_mma(s2[0], a2, b[2], b[3]);
                }
            }
            if (kk < D) {  // D is a multiple of 16: one slice of 16 columns is left
                uint32_t a[4], b[4];
                lm_ldmatrix_x4(qa + kk * 2, a);
                if (NJ == 2) {
                    lm_ldmatrix_x4(kb + kk * 2, b);
                    lm_mma(s[0], a, b[0], b[1]);
                    lm_mma(s[NJ - 1], a, b[2], b[3]);
                } else {
                    // (lanes 16..31 would address columns past the slice: they re-read the first two octets)
                    const uint32_t addr = kst + (uint32_t)(((warp * KW + (lane & 7)) * DS + kk + 8 * ((lane >> 3) & 1)) * 2);
                    lm_ldmatrix_x4(addr, b);
                    lm_mma(s[0], a, b[0], b[1]);
                }
            }
#pragma unroll
            for (int j = 0; j < NJ; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] += s2[j][e];
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < NJ; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = k0 + warp * KW + j * 8 + 2 * tq + (e & 1);
                    s[j][e] = key < k_hi ? s[j][e] * scale_log2 : -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                if (tq == 0) smax[warp * 16 + g + 8 * r] = mx[r];
            }
            __syncthreads();
            float alpha[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float mt = smax[g + 8 * r];
#pragma unroll
                for (int w = 1; w < W; ++w) mt = fmaxf(mt, smax[w * 16 + g + 8 * r]);
                const float m_new = fmaxf(m_run[r], mt);  // finite: key k0 of the tile is visible
                alpha[r] = exp2f(m_run[r] - m_new);
                m_run[r] = m_new;
            }
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                float p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    p[e] = exp2f(s[j][e] - m_run[e >> 1]);
                    sum[e >> 1] += p[e];
                }
                const int col = warp * KW + j * 8 + 2 * tq;
                *reinterpret_cast<__nv_bfloat162*>(Ps + g * PS + col) = __floats2bfloat162_rn(p[0], p[1]);
                *reinterpret_cast<__nv_bfloat162*>(Ps + (g + 8) * PS + col) = __floats2bfloat162_rn(p[2], p[3]);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
                if (tq == 0) ssum[warp * 16 + g + 8 * r] = sum[r];
            }
            __syncthreads();
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float st = 0.f;
#pragma unroll
                for (int w = 0; w < W; ++w) st += ssum[w * 16 + g + 8 * r];
                l_run[r] = l_run[r] * alpha[r] + st;
            }
#pragma unroll
            for (int i = 0; i < NTW; ++i) {
                o[i][0] *= alpha[0];
                o[i][1] *= alpha[0];
                o[i][2] *= alpha[1];
                o[i][3] *= alpha[1];
            }
            // O += P K[:, my columns]
#pragma unroll
            for (int kk2 = 0; kk2 < LM_KT; kk2 += 16) {
                uint32_t a[4];
                lm_ldmatrix_x4(ps_addr + (uint32_t)((a_row * PS + kk2 + a_col) * 2), a);
#pragma unroll
                for (int i = 0; i < NTW; ++i) {
                    if (i < ntw) {
                        uint32_t b0, b1;
                        lm_ldmatrix_x2_trans(kst + (uint32_t)(((kk2 + v_row) * DS + col0 + i * 8) * 2), b0, b1);
                        lm_mma(o[i], a, b0, b1);
                    }
                }
            }
            __syncthreads();  // the tile and Ps are free for the next round
        }
    }
    // results: rows g and g + 8 of this lane, columns col0 + 8 i + 2 tq, + 1
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int h = h0 + g + 8 * r;
        if (h >= H) continue;
        if (splits == 1) {
            const float inv = 1.f / l_run[r];
            bf16* dst = out + ((size_t)h * num_tokens + t) * R;
#pragma unroll
            for (int i = 0; i < NTW; ++i)
                if (i < ntw)
                    *reinterpret_cast<__nv_bfloat162*>(dst + col0 + i * 8 + 2 * tq) =
                        __floats2bfloat162_rn(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
        } else {
            float* dst = partial + (((size_t)t * H + h) * splits + sp) * (R + 2);
#pragma unroll
            for (int i = 0; i < NTW; ++i)
                if (i < ntw) {
                    dst[col0 + i * 8 + 2 * tq] = o[i][2 * r];
                    dst[col0 + i * 8 + 2 * tq + 1] = o[i][2 * r + 1];
                }
            if (warp == 0 && tq == 0) {
                // the merge kernel works in natural-log units
                dst[R] = m_run[r] * 0.6931471805599453f;
                dst[R + 1] = l_run[r];
            }
        }
    }
}

bool latent_mma_supported(int R, int P, const void* qlat, const void* qrot, int q_row_stride, int q_head_stride,
                          const void* pages) {
    const int D = R + P;
    if (R % 32 || P % 16 || R > 512 || R < 32) return false;
    if ((reinterpret_cast<uintptr_t>(pages) & 15) || (reinterpret_cast<uintptr_t>(qlat) & 3) ||
        (reinterpret_cast<uintptr_t>(qrot) & 3) || (q_row_stride & 1) || (q_head_stride & 1))
        return false;
    const size_t smem = (size_t)(16 + LM_KT) * (D + LM_PAD) * 2 + 16 * (LM_KT + LM_PAD) * 2 + 2 * 8 * 16 * 4;
    return smem <= 220 * 1024;
}

template <int NTW, int W>
static int launch_latent_mma(const void* qlat, const void* qrot, int q_row_stride, int q_head_stride,
                             const void* pages, const int* block_tables, int bt_stride, int page_size,
                             const int* positions, const int* row_of_token, void* out, float* partial,
                             int num_tokens, int H, int R, int P, float scale, int splits, cudaStream_t stream) {
    const int D = R + P;
    // Two stages where two blocks of them still share an SM (about 110 KB each).  Otherwise one stage
    // when the grid can fill every SM with two blocks twice over (prompt steps: 0.95 -> 0.74 ms at 2048
    // tokens, 16 heads, 512 + 64 numbers per key), two stages when blocks are few (decode steps, where
    // a block alone on its SM has nothing else to hide the copy behind: 68 us against 84 at 64 rows).
    auto bytes = [&](int st) {
        return (size_t)(16 + st * LM_KT) * (D + LM_PAD) * 2 + 16 * (LM_KT + LM_PAD) * 2 + 2 * W * 16 * 4;
    };
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    const long long blocks = (long long)num_tokens * splits * ((H + 15) / 16);
    const int stages = (bytes(2) <= 110 * 1024 || blocks < 4LL * sms) ? 2 : 1;
    const size_t smem = bytes(stages);
    auto kern = latent_attention_mma_kernel<NTW, W>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return EMS_ERR_LAUNCH;
    }
    dim3 grid(num_tokens, splits, (H + 15) / 16);
    kern<<<grid, W * 32, smem, stream>>>((const bf16*)qlat, (const bf16*)qrot, q_row_stride, q_head_stride,
                                                (const bf16*)pages, block_tables, bt_stride, page_size, positions,
                                                row_of_token, (bf16*)out, partial, num_tokens, H, R, P,
                                                scale * 1.4426950408889634f, splits, stages);
    return launch_status();
}

int run_latent_mma(const void* qlat, const void* qrot, int q_row_stride, int q_head_stride, const void* pages,
                   const int* block_tables, int bt_stride, int page_size, const int* positions,
                   const int* row_of_token, void* out, float* partial, int num_tokens, int H, int R, int P,
                   float scale, int splits, cudaStream_t stream) {
#define EMS_LM(N, W)                                                                                             \
    return launch_latent_mma<N, W>(qlat, qrot, q_row_stride, q_head_stride, pages, block_tables, bt_stride,     \
                                   page_size, positions, row_of_token, out, partial, num_tokens, H, R, P, scale, \
                                   splits, stream)
    // eight warps where every warp still owns whole 8-column tiles of O (R a multiple of 64) and the
    // latent is long enough to keep them busy; four otherwise
    if (R % 64 == 0 && R >= 256) {
        if (R <= 256) EMS_LM(4, 8);
        EMS_LM(8, 8);
    }
    if (R <= 128) EMS_LM(4, 4);
    if (R <= 256) EMS_LM(8, 4);
    EMS_LM(16, 4);
#undef EMS_LM
}

}  // namespace ems
