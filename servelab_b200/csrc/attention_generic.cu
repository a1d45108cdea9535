// Plain paged attention: any head size up to 256, any number of heads and groups,
// any page size, any mix of prompt portions and single decoded tokens, float32
// arithmetic throughout (inputs and outputs float32 or bfloat16).
//
// It is the attention of the 32-bit path and the plain kernel that stands beside
// the fast bfloat16 kernels (which are checked against it).
//
// Work unit: (tile of 32 query rows, kv head).  The query rows of one request and
// one kv head are flattened as rho = local_token * g + head_in_group, so that the
// g query heads sharing a kv head also share each loaded key/value tile.  Keys are
// visited in tiles of 32 aligned to absolute positions, in increasing order, with
// an online softmax per row (running max m, running sum l, float32 accumulator).
// A row's result therefore depends only on that row's query and the keys it may
// see: not on the other rows of the tile, not on how the prompt was cut, and not
// on which pages hold the keys.
//
// Masking: key position r is visible to a query at position a iff r <= a and, with
// a window w > 0, a - r < w.  The position of local token i of a request is
// ctx_len - q_len + i.
//
// Two optional steps for mixers whose scores and weights are modified:
//   * a distance bias: r1_h * ln(1 + r2_h * (a - r)) is subtracted from the scaled score
//     (bias_r1 / bias_r2 hold a pair of numbers per query head; null: none);
//   * every (query head, value head) pair (`pair_out` not null): the grid's z index names the
//     kv head whose VALUES the softmax weights of this block's query heads are applied to,
//     and the result goes, in float32, to pair_out[token][query head][value head][D].  A
//     mixer that mixes the heads' weights after the softmax needs exactly these: mixing the
//     weights and then applying them to a head's values equals mixing these results
//     (slb_mix_heads_gate below).
//
// Reference analogue: the per-sequence torch loop (servelab/parallel/
// tp_model.py:136-157): gather rows by block table, repeat_interleave for the
// groups, float32 scores * D^-1/2, causal mask, float32 softmax, float32 P.V.
#include "common.cuh"

#define AG_BM 32
#define AG_BN 32
#define AG_THREADS 256
#define AG_MAX_D 256

// 0, or 1 once a block-table entry pointed outside the cache (page >= num_pages): those keys
// were read as zeros instead of from outside the pool.
SLB_DEFINE_STATUS_WORD(generic_attention_status_word, slb_paged_attention_generic_status)

template <typename T>
__global__ void __launch_bounds__(AG_THREADS) paged_attention_generic_kernel(
    const T* __restrict__ q, int ldq, const T* __restrict__ kc, const T* __restrict__ vc,
    T* __restrict__ out, int ldo, const int* __restrict__ block_table, int max_pages,
    const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
    const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
    int H, int Hkv, int D, int ps, int num_pages, float scale, int window,
    const float* __restrict__ bias_r1, const float* __restrict__ bias_r2,
    float* __restrict__ pair_out) {
    extern __shared__ float smem[];
    pdl_wait();
    const int ldd = D + 1;
    float* Qs = smem;
    float* Ks = Qs + AG_BM * ldd;
    float* Vs = Ks + AG_BN * ldd;
    float* Ps = Vs + AG_BN * ldd;                 // [AG_BM][AG_BN + 1]

    const int tid = threadIdx.x;
    const int kvh = blockIdx.y;
    const int vh = pair_out != nullptr ? blockIdx.z : kvh;     // the kv head whose values are used
    const int s = tile_seq[blockIdx.x];
    const int row0 = tile_row0[blockIdx.x];
    const int g = H / Hkv;
    const int q0 = cu_q[s];
    const int qlen = cu_q[s + 1] - q0;
    const int ctx = ctx_len[s];
    const int nrows = min(AG_BM, qlen * g - row0);
    if (nrows <= 0) return;
    const int pos_base = ctx - qlen;

    for (int idx = tid; idx < AG_BM * D; idx += AG_THREADS) {
        const int r = idx / D, d = idx - r * D;
        float v = 0.f;
        if (r < nrows) {
            const int rho = row0 + r;
            const int tl = rho / g, hg = rho - tl * g;
            v = to_float(q[(size_t)(q0 + tl) * ldq + (size_t)(kvh * g + hg) * D + d]);
        }
        Qs[r * ldd + d] = v;
    }

    const int r = tid >> 3, c0 = tid & 7;
    const bool row_valid = r < nrows;
    const int my_pos = row_valid ? pos_base + (row0 + r) / g : -1;
    float r1 = 0.f, r2 = 0.f;
    if (bias_r1 != nullptr && row_valid) {
        const int head = kvh * g + (row0 + r) % g;
        r1 = bias_r1[head];
        r2 = bias_r2[head];
    }
    const int p_first = pos_base + row0 / g;
    const int p_last = pos_base + (row0 + nrows - 1) / g;
    int kbeg = 0;
    if (window > 0) kbeg = max(0, p_first - window + 1) / AG_BN * AG_BN;
    const int kend = p_last + 1;
    const int nj = (D + 7) >> 3;

    float m = -INFINITY, l = 0.f;
    float acc[AG_MAX_D / 8];
#pragma unroll
    for (int j = 0; j < AG_MAX_D / 8; ++j) acc[j] = 0.f;

    const int* table = block_table + (size_t)s * max_pages;
    for (int k0 = kbeg; k0 < kend; k0 += AG_BN) {
        __syncthreads();
        for (int idx = tid; idx < AG_BN * D; idx += AG_THREADS) {
            const int kr = idx / D, d = idx - kr * D;
            const int kp = k0 + kr;
            float kv = 0.f, vv = 0.f;
            if (kp < kend) {
                const int page = table[kp / ps];
                if (page >= num_pages) {
                    atomicCAS(&generic_attention_status_word, 0, 1);
                } else if (page >= 0) {
                    const size_t slot = (size_t)page * Hkv * ps + kp % ps;
                    kv = to_float(kc[(slot + (size_t)kvh * ps) * D + d]);
                    vv = to_float(vc[(slot + (size_t)vh * ps) * D + d]);
                }
            }
            Ks[kr * ldd + d] = kv;
            Vs[kr * ldd + d] = vv;
        }
        __syncthreads();

        float sc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int d = 0; d < D; ++d) {
            const float qv = Qs[r * ldd + d];
#pragma unroll
            for (int j = 0; j < 4; ++j) sc[j] += qv * Ks[(c0 + 8 * j) * ldd + d];
        }
        float tmax = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kp = k0 + c0 + 8 * j;
            const bool vis = row_valid && kp <= my_pos && (window <= 0 || my_pos - kp < window);
            sc[j] = vis ? sc[j] * scale - (bias_r1 != nullptr ? r1 * logf(1.f + r2 * (float)(my_pos - kp)) : 0.f)
                        : -INFINITY;
            tmax = fmaxf(tmax, sc[j]);
        }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
        const float m_new = fmaxf(m, tmax);
        float alpha = 1.f, psum = 0.f;
        float p[4] = {0.f, 0.f, 0.f, 0.f};
        if (m_new != -INFINITY) {
            alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                p[j] = (sc[j] == -INFINITY) ? 0.f : expf(sc[j] - m_new);
                psum += p[j];
            }
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        psum += __shfl_xor_sync(0xffffffffu, psum, 4);
        l = l * alpha + psum;
        m = m_new;
#pragma unroll
        for (int j = 0; j < 4; ++j) Ps[r * (AG_BN + 1) + c0 + 8 * j] = p[j];
        __syncwarp();                              // a row's 8 threads share a warp

#pragma unroll
        for (int j = 0; j < AG_MAX_D / 8; ++j) acc[j] *= alpha;
        for (int k = 0; k < AG_BN; ++k) {
            const float pv = Ps[r * (AG_BN + 1) + k];
#pragma unroll
            for (int j = 0; j < AG_MAX_D / 8; ++j) {
                const int c = c0 + 8 * j;
                if (j < nj && c < D) acc[j] += pv * Vs[k * ldd + c];
            }
        }
    }

    if (row_valid) {
        const int rho = row0 + r;
        const int tl = rho / g, hg = rho - tl * g;
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        if (pair_out != nullptr) {
            float* o = pair_out + (((size_t)(q0 + tl) * H + (size_t)(kvh * g + hg)) * Hkv + vh) * D;
#pragma unroll
            for (int j = 0; j < AG_MAX_D / 8; ++j) {
                const int c = c0 + 8 * j;
                if (j < nj && c < D) o[c] = acc[j] * inv;
            }
            return;
        }
        T* o = out + (size_t)(q0 + tl) * ldo + (size_t)(kvh * g + hg) * D;
#pragma unroll
        for (int j = 0; j < AG_MAX_D / 8; ++j) {
            const int c = c0 + 8 * j;
            if (j < nj && c < D) o[c] = from_float<T>(acc[j] * inv);
        }
    }
}

template <typename T>
static int launch_generic(const T* q, int ldq, const T* kc, const T* vc, T* out, int ldo,
                          const int* block_table, int max_pages, const int* cu_q,
                          const int* ctx_len, const int* tile_seq, const int* tile_row0,
                          int num_tiles, int H, int Hkv, int D, int ps, int num_pages, float scale,
                          int window, const float* bias_r1, const float* bias_r2, float* pair_out,
                          cudaStream_t st) {
    if (num_tiles <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || D <= 0 || ps <= 0 || max_pages <= 0 || num_pages <= 0)
        return SLB_ERR_BAD_ARG;
    if ((bias_r1 == nullptr) != (bias_r2 == nullptr)) return SLB_ERR_BAD_ARG;
    if (D > AG_MAX_D || Hkv > 65535) return SLB_ERR_TOO_LARGE;
    const size_t smem = ((size_t)(AG_BM + 2 * AG_BN) * (D + 1) + AG_BM * (AG_BN + 1)) * sizeof(float);
    // the largest this kernel can ask for (head size AG_MAX_D), set once per device
    constexpr size_t SMEM_MAX = ((size_t)(AG_BM + 2 * AG_BN) * (AG_MAX_D + 1) + AG_BM * (AG_BN + 1)) * sizeof(float);
    static unsigned long long configured = 0;     // per template instance, a bit per device
    const int rc = slb_configure(&configured, paged_attention_generic_kernel<T>, SMEM_MAX);
    if (rc != 0) return rc;
    return slb_launch(paged_attention_generic_kernel<T>, dim3(num_tiles, Hkv, pair_out != nullptr ? Hkv : 1),
                      dim3(AG_THREADS), smem, st, q, ldq, kc, vc, out, ldo, block_table, max_pages, cu_q,
                      ctx_len, tile_seq, tile_row0, H, Hkv, D, ps, num_pages, scale, window, bias_r1,
                      bias_r2, pair_out);
}

// What follows the attention of a mixer with mixed heads and an output gate, in one pass:
//   out[t][h][d] = (sum_g talk[h][g] * pairs[t][g][c(h)][d]) * sigmoid(gate[t][h][d])
// `pairs` (float32) holds, per query head g, its softmax weights applied to the values of
// nvh kv heads: nvh = Hkv (every pair; c(h) is h's kv head) or 1 (each head's own kv head only,
// which is all an unmixed mixer needs; talk must then be null).  With `pair_ml` the pairs are
// the unnormalised partials of `splits` key ranges, pairs[t][g][c][split][d], with their running
// maxima (base-2 domain) and sums in pair_ml[t][g][c][split][2]: the splits are combined here,
// weight 2^(m_split - M) / L each.  `pairs` may be null: then `direct` [T, H D] (type T) is the
// attention's plain result and only the gate is applied; `talk` and `gate` may each be null.
// A block owns one token and one kv head c, whose group of query heads it finishes MIX_HEADS at
// a time.  A thread owns VEC neighbouring columns d and a slice of the source heads q: it reads
// pairs[t][q][c][d] once per q of its slice (combining the splits), multiplies by the mixing
// weights of the heads being finished, and the slices are added up through shared memory -- a
// step of few tokens has little work, and many short chains of loads finish sooner than few
// long ones.
#define MIX_HEADS 4
#define MIX_THREADS 256
#define MIX_ROWS_FROM 64             // above this many tokens the unsliced kernel below runs

template <typename T, int VEC>
__global__ void __launch_bounds__(MIX_THREADS) mix_heads_gate_kernel(
    const float* __restrict__ pairs, const float* __restrict__ pair_ml, int splits, int nvh,
    const T* direct, int ldi, const float* __restrict__ talk, const T* __restrict__ gate, int ldg,
    T* out, int ldo, int H, int Hkv, int D) {
    extern __shared__ float mix_smem[];
    const int dv = D / VEC;                        // column groups
    const int slices = max(1, min(MIX_THREADS / dv, H));
    float* red = mix_smem;                         // [slices][MIX_HEADS][D]
    float* talk_s = red + slices * MIX_HEADS * D;  // [H][H] (with talk)
    float* factor = talk_s + (talk != nullptr ? H * H : 0);     // [H][nvh][splits] (with pair_ml)
    if (talk != nullptr)
        for (int i = threadIdx.x; i < H * H; i += blockDim.x) talk_s[i] = talk[i];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y, c = blockIdx.x;
    const int ci = nvh > 1 ? c : 0;
    if (pair_ml != nullptr) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {          // (q, ci) of every source head
            const float* ml = pair_ml + (((size_t)t * H + i) * nvh + ci) * splits * 2;
            float M = -INFINITY;
            for (int sp = 0; sp < splits; ++sp) M = fmaxf(M, ml[2 * sp]);
            float L = 0.f;
            for (int sp = 0; sp < splits; ++sp)
                if (ml[2 * sp] != -INFINITY) L += ml[2 * sp + 1] * exp2f(ml[2 * sp] - M);
            for (int sp = 0; sp < splits; ++sp)
                factor[i * splits + sp] = (L > 0.f && ml[2 * sp] != -INFINITY) ? exp2f(ml[2 * sp] - M) / L : 0.f;
        }
    }
    __syncthreads();
    const int g = H / Hkv;
    const int dcol = threadIdx.x % dv, slice = threadIdx.x / dv;
    const int d = dcol * VEC;
    const bool worker = slice < slices;
    for (int h0 = c * g; h0 < (c + 1) * g; h0 += MIX_HEADS) {
        const int nh = min(MIX_HEADS, (c + 1) * g - h0);
        float acc[MIX_HEADS][VEC];
#pragma unroll
        for (int i = 0; i < MIX_HEADS; ++i)
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[i][v] = 0.f;
        if (worker && pairs == nullptr) {
            if (slice == 0) {
#pragma unroll
                for (int i = 0; i < MIX_HEADS; ++i)
#pragma unroll
                    for (int v = 0; v < VEC; ++v)
                        if (i < nh) acc[i][v] = to_float(direct[(size_t)t * ldi + (size_t)(h0 + i) * D + d + v]);
            }
        } else if (worker) {
            // without talk, head h needs only its own result
            const int q_lo = talk != nullptr ? 0 : h0, q_hi = talk != nullptr ? H : h0 + nh;
            for (int q = q_lo + slice; q < q_hi; q += slices) {
                const size_t pi = ((size_t)t * H + q) * nvh + ci;
                float p[VEC];
#pragma unroll
                for (int v = 0; v < VEC; ++v) p[v] = 0.f;
                if (pair_ml != nullptr) {
#pragma unroll 4
                    for (int sp = 0; sp < splits; ++sp) {
                        const float f = factor[q * splits + sp];
                        const float* src = pairs + (pi * splits + sp) * D + d;
                        if constexpr (VEC == 4) {
                            const float4 x = *reinterpret_cast<const float4*>(src);
                            p[0] += f * x.x; p[1] += f * x.y; p[2] += f * x.z; p[3] += f * x.w;
                        } else {
                            p[0] += f * src[0];
                        }
                    }
                } else {
                    const float* src = pairs + pi * D + d;
                    if constexpr (VEC == 4) {
                        const float4 x = *reinterpret_cast<const float4*>(src);
                        p[0] = x.x; p[1] = x.y; p[2] = x.z; p[3] = x.w;
                    } else {
                        p[0] = src[0];
                    }
                }
#pragma unroll
                for (int i = 0; i < MIX_HEADS; ++i) {
                    const float w = talk != nullptr ? (i < nh ? talk_s[(h0 + i) * H + q] : 0.f)
                                                    : (h0 + i == q ? 1.f : 0.f);
#pragma unroll
                    for (int v = 0; v < VEC; ++v) acc[i][v] = fmaf(w, p[v], acc[i][v]);
                }
            }
        }
        if (worker) {
#pragma unroll
            for (int i = 0; i < MIX_HEADS; ++i)
#pragma unroll
                for (int v = 0; v < VEC; ++v) red[(slice * MIX_HEADS + i) * D + d + v] = acc[i][v];
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nh * D; idx += blockDim.x) {
            const int i = idx / D, dd = idx - i * D;
            float r = 0.f;
            for (int sl = 0; sl < slices; ++sl) r += red[(sl * MIX_HEADS + i) * D + dd];
            const size_t col = (size_t)(h0 + i) * D + dd;
            if (gate != nullptr) r *= 1.f / (1.f + expf(-to_float(gate[(size_t)t * ldg + col])));
            out[(size_t)t * ldo + col] = from_float<T>(r);
        }
        __syncthreads();                           // red is rewritten by the next group of heads
    }
}

// The same arithmetic for steps of many tokens, where there is work enough without slicing: a
// thread owns one kv head c and VEC neighbouring columns d of a token, reads pairs[t][q][c][d] once
// for every source head q and finishes, MIX_ROW_HEADS at a time, the heads of group c from it.
#define MIX_ROW_HEADS 8

template <typename T, int VEC>
__global__ void __launch_bounds__(256) mix_heads_gate_rows_kernel(
    const float* __restrict__ pairs, const float* __restrict__ pair_ml, int splits, int nvh,
    const T* direct, int ldi, const float* __restrict__ talk, const T* __restrict__ gate, int ldg,
    T* out, int ldo, int H, int Hkv, int D) {
    extern __shared__ float mix_smem[];
    float* talk_s = mix_smem;                      // [H][H] (with talk)
    float* factor = mix_smem + (talk != nullptr ? H * H : 0);   // [H][nvh][splits] (with pair_ml)
    if (talk != nullptr)
        for (int i = threadIdx.x; i < H * H; i += blockDim.x) talk_s[i] = talk[i];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y;
    if (pair_ml != nullptr) {
        for (int i = threadIdx.x; i < H * nvh; i += blockDim.x) {
            const float* ml = pair_ml + ((size_t)t * H * nvh + i) * splits * 2;
            float M = -INFINITY;
            for (int sp = 0; sp < splits; ++sp) M = fmaxf(M, ml[2 * sp]);
            float L = 0.f;
            for (int sp = 0; sp < splits; ++sp)
                if (ml[2 * sp] != -INFINITY) L += ml[2 * sp + 1] * exp2f(ml[2 * sp] - M);
            for (int sp = 0; sp < splits; ++sp)
                factor[i * splits + sp] = (L > 0.f && ml[2 * sp] != -INFINITY) ? exp2f(ml[2 * sp] - M) / L : 0.f;
        }
    }
    __syncthreads();
    const int g = H / Hkv;
    const int dv = D / VEC;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= Hkv * dv) return;
    const int c = idx / dv, d = (idx - c * dv) * VEC;       // the kv head whose group is finished, columns
    for (int h0 = c * g; h0 < (c + 1) * g; h0 += MIX_ROW_HEADS) {
        const int nh = min(MIX_ROW_HEADS, (c + 1) * g - h0);
        float acc[MIX_ROW_HEADS][VEC];
#pragma unroll
        for (int i = 0; i < MIX_ROW_HEADS; ++i)
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[i][v] = 0.f;
        if (pairs == nullptr) {
#pragma unroll
            for (int i = 0; i < MIX_ROW_HEADS; ++i)
#pragma unroll
                for (int v = 0; v < VEC; ++v)
                    if (i < nh) acc[i][v] = to_float(direct[(size_t)t * ldi + (size_t)(h0 + i) * D + d + v]);
        } else {
            const int ci = nvh > 1 ? c : 0;
            // without talk, head h needs only its own result
            const int q_lo = talk != nullptr ? 0 : h0, q_hi = talk != nullptr ? H : h0 + nh;
            for (int q = q_lo; q < q_hi; ++q) {
                const size_t pi = ((size_t)t * H + q) * nvh + ci;
                float p[VEC];
#pragma unroll
                for (int v = 0; v < VEC; ++v) p[v] = 0.f;
                if (pair_ml != nullptr) {
                    for (int sp = 0; sp < splits; ++sp) {
                        const float f = factor[(q * nvh + ci) * splits + sp];
                        const float* src = pairs + (pi * splits + sp) * D + d;
                        if constexpr (VEC == 4) {
                            const float4 x = *reinterpret_cast<const float4*>(src);
                            p[0] += f * x.x; p[1] += f * x.y; p[2] += f * x.z; p[3] += f * x.w;
                        } else {
                            p[0] += f * src[0];
                        }
                    }
                } else {
                    const float* src = pairs + pi * D + d;
                    if constexpr (VEC == 4) {
                        const float4 x = *reinterpret_cast<const float4*>(src);
                        p[0] = x.x; p[1] = x.y; p[2] = x.z; p[3] = x.w;
                    } else {
                        p[0] = src[0];
                    }
                }
#pragma unroll
                for (int i = 0; i < MIX_ROW_HEADS; ++i) {
                    const float w = talk != nullptr ? (i < nh ? talk_s[(h0 + i) * H + q] : 0.f)
                                                    : (h0 + i == q ? 1.f : 0.f);
#pragma unroll
                    for (int v = 0; v < VEC; ++v) acc[i][v] = fmaf(w, p[v], acc[i][v]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < MIX_ROW_HEADS; ++i) {
            if (i >= nh) break;
            const size_t col = (size_t)(h0 + i) * D + d;
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                float r = acc[i][v];
                if (gate != nullptr) r *= 1.f / (1.f + expf(-to_float(gate[(size_t)t * ldg + col + v])));
                out[(size_t)t * ldo + col + v] = from_float<T>(r);
            }
        }
    }
}

template <typename T>
static int launch_mix(const float* pairs, const float* pair_ml, int splits, int nvh, const T* direct,
                      int ldi, const float* talk, const T* gate, int ldg, T* out, int ldo, int T_tokens,
                      int H, int Hkv, int D, cudaStream_t st) {
    if (T_tokens <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || D <= 0 || T_tokens > 65535 || Hkv > 65535 ||
        (pairs == nullptr) == (direct == nullptr))
        return SLB_ERR_BAD_ARG;
    if (pairs != nullptr && ((nvh != 1 && nvh != Hkv) || (talk != nullptr && nvh != Hkv && Hkv != 1)))
        return SLB_ERR_BAD_ARG;
    if (pair_ml != nullptr && (pairs == nullptr || splits < 1)) return SLB_ERR_BAD_ARG;
    if (D > AG_MAX_D) return SLB_ERR_TOO_LARGE;
    const bool vec = D % 4 == 0 && ((uintptr_t)pairs & 15) == 0 && pairs != nullptr;
    const int dv = vec ? D / 4 : D;
    if (T_tokens > MIX_ROWS_FROM) {                    // many tokens: a thread a (kv head, columns) pair
        const size_t smem_rows = ((talk != nullptr ? (size_t)H * H : 0) +
                                  (pair_ml != nullptr ? (size_t)H * nvh * splits : 0)) * sizeof(float);
        if (smem_rows <= 48 * 1024) {
            const int work = Hkv * dv;
            const int threads = work >= 256 ? 256 : (work + 31) / 32 * 32;
            const dim3 grid_rows((work + threads - 1) / threads, T_tokens);
            if (vec)
                return slb_launch(mix_heads_gate_rows_kernel<T, 4>, grid_rows, dim3(threads), smem_rows, st, pairs,
                                  pair_ml, splits, nvh, direct, ldi, talk, gate, ldg, out, ldo, H, Hkv, D);
            return slb_launch(mix_heads_gate_rows_kernel<T, 1>, grid_rows, dim3(threads), smem_rows, st, pairs,
                              pair_ml, splits, nvh, direct, ldi, talk, gate, ldg, out, ldo, H, Hkv, D);
        }
    }
    const int slices = MIX_THREADS / dv < 1 ? 1 : (MIX_THREADS / dv < H ? MIX_THREADS / dv : H);
    const size_t smem = ((size_t)slices * MIX_HEADS * D + (talk != nullptr ? (size_t)H * H : 0) +
                         (pair_ml != nullptr ? (size_t)H * splits : 0)) * sizeof(float);
    constexpr size_t SMEM_MAX = 96 * 1024;
    if (smem > SMEM_MAX) return SLB_ERR_TOO_LARGE;
    static unsigned long long configured[2] = {0, 0};  // per template instance, a bit per device
    const dim3 grid(Hkv, T_tokens);
    if (vec) {
        const int rc = slb_configure(&configured[0], mix_heads_gate_kernel<T, 4>, SMEM_MAX);
        if (rc != 0) return rc;
        return slb_launch(mix_heads_gate_kernel<T, 4>, grid, dim3(MIX_THREADS), smem, st, pairs, pair_ml, splits,
                          nvh, direct, ldi, talk, gate, ldg, out, ldo, H, Hkv, D);
    }
    const int rc = slb_configure(&configured[1], mix_heads_gate_kernel<T, 1>, SMEM_MAX);
    if (rc != 0) return rc;
    return slb_launch(mix_heads_gate_kernel<T, 1>, grid, dim3(MIX_THREADS), smem, st, pairs, pair_ml, splits, nvh,
                      direct, ldi, talk, gate, ldg, out, ldo, H, Hkv, D);
}

extern "C" {
int slb_paged_attention_generic_f32(const float* q, int ldq, const float* kc, const float* vc,
                                    float* out, int ldo, const int* block_table, int max_pages,
                                    const int* cu_q, const int* ctx_len, const int* tile_seq,
                                    const int* tile_row0, int num_tiles, int H, int Hkv, int D,
                                    int ps, int num_pages, float scale, int window, const float* bias_r1,
        const float* bias_r2, float* pair_out, cudaStream_t st) {
    return launch_generic<float>(q, ldq, kc, vc, out, ldo, block_table, max_pages, cu_q, ctx_len,
                                 tile_seq, tile_row0, num_tiles, H, Hkv, D, ps, num_pages, scale, window,
                                 bias_r1, bias_r2, pair_out, st);
}
int slb_paged_attention_generic_bf16(const bf16* q, int ldq, const bf16* kc, const bf16* vc,
                                     bf16* out, int ldo, const int* block_table, int max_pages,
                                     const int* cu_q, const int* ctx_len, const int* tile_seq,
                                     const int* tile_row0, int num_tiles, int H, int Hkv, int D,
                                     int ps, int num_pages, float scale, int window, const float* bias_r1,
        const float* bias_r2, float* pair_out, cudaStream_t st) {
    return launch_generic<bf16>(q, ldq, kc, vc, out, ldo, block_table, max_pages, cu_q, ctx_len,
                                 tile_seq, tile_row0, num_tiles, H, Hkv, D, ps, num_pages, scale, window,
                                 bias_r1, bias_r2, pair_out, st);
}
int slb_mix_heads_gate_f32(const float* pairs, const float* pair_ml, int splits, int nvh,
                           const float* direct, int ldi, const float* talk, const float* gate, int ldg,
                           float* out, int ldo, int T_tokens, int H, int Hkv, int D, cudaStream_t st) {
    return launch_mix<float>(pairs, pair_ml, splits, nvh, direct, ldi, talk, gate, ldg, out, ldo, T_tokens,
                             H, Hkv, D, st);
}
int slb_mix_heads_gate_bf16(const float* pairs, const float* pair_ml, int splits, int nvh,
                            const bf16* direct, int ldi, const float* talk, const bf16* gate, int ldg,
                            bf16* out, int ldo, int T_tokens, int H, int Hkv, int D, cudaStream_t st) {
    return launch_mix<bf16>(pairs, pair_ml, splits, nvh, direct, ldi, talk, gate, ldg, out, ldo, T_tokens,
                            H, Hkv, D, st);
}
// rows per tile of the generic kernel (the host builds the tile list with it)
int slb_paged_attention_generic_tile_rows() { return AG_BM; }
}
