// The mixed-head attention of attention_mixed.cu on the tensor cores, for the bfloat16
// engine: scores, the mixing of the heads' weights and the weighted sum of the values are
// all mma.sync products with float32 accumulators.
//
// A block takes 16 query tokens with all their heads and walks the keys twice in tiles of
// 32, as the CUDA-core kernel does (first each row's maximum and sum, then the finished
// weights). Head h belongs to warp h mod (number of warps). Per tile of the second walk:
//   1. S_h = Q_h K^T on the tensor cores (bfloat16 operands are exact, float32 sums),
//      w_h = exp(S_h * scale - max_h) / sum_h in float32 registers;
//   2. every weight is split w = hi + lo into two bfloat16 numbers (|lo| <= 2^-9 |w|, what is
//      left is below 2^-17 |w|) and written position-major, [token, key][head];
//   3. the heads are mixed as a product over the head index, W' = M W: M (bfloat16 in the
//      checkpoint, so exact) times hi and times lo, summed in float32; the result, split
//      again, goes back head-major, [head][token][key];
//   4. O_h += W'_h V on the tensor cores, hi and lo in turn, from a transposed value tile.
// So the weights keep 16 bits of mantissa through both products, against the 8 that the
// values they multiply have. The float32 engine never comes here.
#include "common.cuh"

namespace mb {

struct MixedAttentionArgs {     // the same structure as in attention_mixed.cu
    const void* qkv;
    int row_width;
    const void* k_pages;
    const void* v_pages;
    const int* table;
    int max_pages;
    const int* q_start;
    const int* kv_len;
    const float* mix;
    void* out;
    int n_q, n_kv, d, vd, page_size;
    float scale;
    int window, tiles_per_seq, bq;
    int num_splits, mode;
    float* part_ml;
    float* part_out;
};

typedef __nv_bfloat16 bf;
constexpr int MM_ROWS = 16;     // query tokens per block
constexpr int MM_KEYS = 32;     // keys per tile
constexpr int MM_PAD = 8;       // elements of padding per shared-memory row

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t ld32(const bf* p) { return *reinterpret_cast<const uint32_t*>(p); }

__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const bf xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
    const bf xl = __float2bfloat16_rn(x - __bfloat162float(xh));
    const bf yl = __float2bfloat16_rn(y - __bfloat162float(yh));
    hi = (uint32_t)__bfloat16_as_ushort(xh) | ((uint32_t)__bfloat16_as_ushort(yh) << 16);
    lo = (uint32_t)__bfloat16_as_ushort(xl) | ((uint32_t)__bfloat16_as_ushort(yl) << 16);
}

struct MmaLayout {      // offsets in bytes of the shared-memory regions
    int q, k, vt, p_hi, p_lo, m_hi, m_lo, t, pages, total;
};

__host__ __device__ inline MmaLayout mma_layout(int H, int G, int d, int vd) {
    const int Hp = (H + 15) / 16 * 16;
    MmaLayout l;
    int at = 0;
    l.q = at;     at += H * MM_ROWS * (d + MM_PAD) * 2;
    l.k = at;     at += G * MM_KEYS * (d + MM_PAD) * 2;
    l.vt = at;    at += G * vd * (MM_KEYS + MM_PAD) * 2;
    l.p_hi = at;  at += MM_ROWS * MM_KEYS * Hp * 2;
    l.p_lo = at;  at += MM_ROWS * MM_KEYS * Hp * 2;
    l.m_hi = at;  at += Hp * MM_ROWS * (MM_KEYS + MM_PAD) * 2;
    l.m_lo = at;  at += Hp * MM_ROWS * (MM_KEYS + MM_PAD) * 2;
    l.t = at;     at += Hp * Hp * 2;
    l.pages = at; at += MM_KEYS * 4;
    l.total = at;
    return l;
}

template <int NW, int HPW, int NV>
__global__ void __launch_bounds__(NW * 32)
mixed_head_attention_mma_kernel(const MixedAttentionArgs a) {
    grid_dependency_sync();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.n_q, G = a.n_kv, d = a.d, vd = a.vd;
    const int R = H / G;
    const int Hp = (H + 15) / 16 * 16;
    const int seq = blockIdx.x / a.tiles_per_seq;
    const int tile = blockIdx.x - seq * a.tiles_per_seq;
    const int q_begin = a.q_start[seq];
    const int q_len = a.q_start[seq + 1] - q_begin;
    const int tok0 = tile * MM_ROWS;
    if (tok0 >= q_len) return;
    const int kv_len = a.kv_len[seq];
    const int first_pos = kv_len - q_len;
    const int n_tok = min(MM_ROWS, q_len - tok0);
    const bf* qkv = reinterpret_cast<const bf*>(a.qkv);
    const bf* k_pages = reinterpret_cast<const bf*>(a.k_pages);
    const bf* v_pages = reinterpret_cast<const bf*>(a.v_pages);

    const MmaLayout L = mma_layout(H, G, d, vd);
    bf* q_s = reinterpret_cast<bf*>(smem_raw + L.q);
    bf* k_s = reinterpret_cast<bf*>(smem_raw + L.k);
    bf* vt_s = reinterpret_cast<bf*>(smem_raw + L.vt);
    bf* p_hi = reinterpret_cast<bf*>(smem_raw + L.p_hi);
    bf* p_lo = reinterpret_cast<bf*>(smem_raw + L.p_lo);
    bf* m_hi = reinterpret_cast<bf*>(smem_raw + L.m_hi);
    bf* m_lo = reinterpret_cast<bf*>(smem_raw + L.m_lo);
    bf* t_s = reinterpret_cast<bf*>(smem_raw + L.t);
    int* page_s = reinterpret_cast<int*>(smem_raw + L.pages);
    const int qs = d + MM_PAD;                 // row strides in elements
    const int ks = MM_KEYS + MM_PAD;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // queries (zeros for rows beyond the tile), the mixing matrix (identity when absent)
    const int chunks = d / 8;
    for (int idx = tid; idx < H * MM_ROWS * chunks; idx += NW * 32) {
        const int ch = idx % chunks, i = (idx / chunks) % MM_ROWS, h = idx / (chunks * MM_ROWS);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (i < n_tok)
            v = *reinterpret_cast<const uint4*>(qkv + (int64_t)(q_begin + tok0 + i) * a.row_width + h * d + ch * 8);
        *reinterpret_cast<uint4*>(q_s + (h * MM_ROWS + i) * qs + ch * 8) = v;
    }
    for (int idx = tid; idx < Hp * Hp; idx += NW * 32) {
        const int h = idx / Hp, gg = idx - h * Hp;
        float v = 0.f;
        if (h < H && gg < H) v = a.mix ? a.mix[h * H + gg] : (h == gg ? 1.f : 0.f);
        t_s[idx] = __float2bfloat16_rn(v);
    }

    const int p_min = first_pos + tok0, p_max = first_pos + tok0 + n_tok - 1;
    int t_lo = 0;
    if (a.window > 0 && p_min - a.window + 1 > 0) t_lo = (p_min - a.window + 1) / MM_KEYS;
    int t_hi = p_max / MM_KEYS + 1;
    if (a.num_splits > 1) {
        const int per = (t_hi - t_lo + a.num_splits - 1) / a.num_splits;
        t_lo += (int)blockIdx.y * per;
        if (t_lo + per < t_hi) t_hi = t_lo + per;
    }

    // rows of this thread: g and g + 8 of the tile
    const bool ok0 = g < n_tok, ok1 = g + 8 < n_tok;
    const int pos0 = first_pos + tok0 + g, pos1 = pos0 + 8;

    float row_m[HPW][2], row_l[HPW][2];
    float acc[HPW][NV][4];
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        row_m[hh][0] = row_m[hh][1] = -INFINITY;
        row_l[hh][0] = row_l[hh][1] = 0.f;
#pragma unroll
        for (int n = 0; n < NV; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[hh][n][e] = 0.f;
    }

    if (a.mode == 2) {
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) {
            const int h = warp + NW * hh;
            if (h >= H) continue;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                if (!(half ? ok1 : ok0)) continue;
                const float* ml = a.part_ml +
                    ((int64_t)(q_begin + tok0 + g + 8 * half) * H + h) * a.num_splits * 2;
                float big = -INFINITY;
                for (int z = 0; z < a.num_splits; ++z) big = fmaxf(big, ml[2 * z]);
                float sum = 0.f;
                for (int z = 0; z < a.num_splits; ++z)
                    if (ml[2 * z] > -INFINITY) sum += ml[2 * z + 1] * expf(ml[2 * z] - big);
                row_m[hh][half] = big;
                row_l[hh][half] = sum;
            }
        }
    }

    const int pass_begin = a.mode == 2 ? 1 : 0, pass_end = a.mode == 1 ? 1 : 2;
    for (int pass = pass_begin; pass < pass_end; ++pass) {
        if (pass == 1) {
#pragma unroll
            for (int hh = 0; hh < HPW; ++hh)
#pragma unroll
                for (int half = 0; half < 2; ++half)
                    row_l[hh][half] = row_l[hh][half] > 0.f ? 1.f / row_l[hh][half] : 0.f;
        }
        for (int kt = t_lo; kt < t_hi; ++kt) {
            __syncthreads();
            if (tid < MM_KEYS) {
                const int key = kt * MM_KEYS + tid;
                int page = -1;
                if (key < kv_len) page = table_page(a.table, seq, a.max_pages, key / a.page_size);
                page_s[tid] = page;
            }
            __syncthreads();
            for (int idx = tid; idx < G * MM_KEYS * chunks; idx += NW * 32) {
                const int ch = idx % chunks, j = (idx / chunks) % MM_KEYS, c = idx / (chunks * MM_KEYS);
                const int page = page_s[j];
                uint4 v = make_uint4(0, 0, 0, 0);
                if (page >= 0) {
                    const int key = kt * MM_KEYS + j;
                    v = *reinterpret_cast<const uint4*>(
                        k_pages + (((int64_t)page * G + c) * a.page_size + (key % a.page_size)) * d + ch * 8);
                }
                *reinterpret_cast<uint4*>(k_s + (c * MM_KEYS + j) * qs + ch * 8) = v;
            }
            if (pass == 1) {
                const int vchunks = vd / 8;
                for (int idx = tid; idx < G * MM_KEYS * vchunks; idx += NW * 32) {
                    const int j = idx % MM_KEYS, ch = (idx / MM_KEYS) % vchunks, c = idx / (MM_KEYS * vchunks);
                    const int page = page_s[j];
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (page >= 0) {
                        const int key = kt * MM_KEYS + j;
                        v = *reinterpret_cast<const uint4*>(
                            v_pages + (((int64_t)page * G + c) * a.page_size + (key % a.page_size)) * vd + ch * 8);
                    }
                    const bf* e = reinterpret_cast<const bf*>(&v);
#pragma unroll
                    for (int x = 0; x < 8; ++x) vt_s[(c * vd + ch * 8 + x) * ks + j] = e[x];
                }
            }
            __syncthreads();

            // 1. scores and weights of this warp's heads
#pragma unroll
            for (int hh = 0; hh < HPW; ++hh) {
                const int h = warp + NW * hh;
                if (h >= H) continue;
                const int c = h / R;
                float s[4][4];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
                const bf* qrow = q_s + (h * MM_ROWS + g) * qs + 2 * t;
                for (int k0 = 0; k0 < d; k0 += 16) {
                    uint32_t af[4];
                    af[0] = ld32(qrow + k0);
                    af[1] = ld32(qrow + 8 * qs + k0);
                    af[2] = ld32(qrow + k0 + 8);
                    af[3] = ld32(qrow + 8 * qs + k0 + 8);
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        const bf* krow = k_s + (c * MM_KEYS + nt * 8 + g) * qs + k0 + 2 * t;
                        mma_16816(s[nt], af, ld32(krow), ld32(krow + 8));
                    }
                }
                // what each element may see
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = nt * 8 + 2 * t + (e & 1);
                        const int key = kt * MM_KEYS + j;
                        const bool second = e >= 2;
                        const int pos = second ? pos1 : pos0;
                        bool seen = (second ? ok1 : ok0) && page_s[j] >= 0 && key <= pos;
                        if (a.window > 0) seen = seen && key > pos - a.window;
                        s[nt][e] = seen ? s[nt][e] * a.scale : -INFINITY;
                        if (second) mx1 = fmaxf(mx1, s[nt][e]); else mx0 = fmaxf(mx0, s[nt][e]);
                    }
                if (pass == 0) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                    const float n0 = fmaxf(row_m[hh][0], mx0), n1 = fmaxf(row_m[hh][1], mx1);
                    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        if (n0 > -INFINITY) sum0 += (s[nt][0] > -INFINITY ? expf(s[nt][0] - n0) : 0.f) +
                                                    (s[nt][1] > -INFINITY ? expf(s[nt][1] - n0) : 0.f);
                        if (n1 > -INFINITY) sum1 += (s[nt][2] > -INFINITY ? expf(s[nt][2] - n1) : 0.f) +
                                                    (s[nt][3] > -INFINITY ? expf(s[nt][3] - n1) : 0.f);
                    }
                    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
                    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
                    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
                    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
                    const float c0 = n0 > -INFINITY ? expf(row_m[hh][0] - n0) : 1.f;
                    const float c1 = n1 > -INFINITY ? expf(row_m[hh][1] - n1) : 1.f;
                    row_l[hh][0] = row_l[hh][0] * c0 + sum0;
                    row_l[hh][1] = row_l[hh][1] * c1 + sum1;
                    row_m[hh][0] = n0;
                    row_m[hh][1] = n1;
                    continue;
                }
                // 2. finished weights, split, position-major
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int half = e >> 1;
                        float p = 0.f;
                        if (s[nt][e] > -INFINITY) p = expf(s[nt][e] - row_m[hh][half]) * row_l[hh][half];
                        const bf ph = __float2bfloat16_rn(p);
                        const bf pl = __float2bfloat16_rn(p - __bfloat162float(ph));
                        const int at = ((g + 8 * half) * MM_KEYS + nt * 8 + 2 * t + (e & 1)) * Hp + h;
                        p_hi[at] = ph;
                        p_lo[at] = pl;
                    }
            }
            if (pass == 0) continue;
            // heads beyond H never write: their columns must read as zero
            if (Hp > H)
                for (int idx = tid; idx < MM_ROWS * MM_KEYS * (Hp - H); idx += NW * 32) {
                    const int at = (idx / (Hp - H)) * Hp + H + idx % (Hp - H);
                    p_hi[at] = __float2bfloat16_rn(0.f);
                    p_lo[at] = __float2bfloat16_rn(0.f);
                }
            __syncthreads();

            // 3. the heads mixed: W'[h][pos] = sum_g M[h][g] W[g][pos]
            for (int ntile = warp; ntile < MM_ROWS * MM_KEYS / 8; ntile += NW) {
                const int pos_b = ntile * 8 + g;          // B operand: column n = g
                for (int mt = 0; mt < Hp / 16; ++mt) {
                    float cm[4] = {0.f, 0.f, 0.f, 0.f};
                    for (int kk = 0; kk < Hp / 16; ++kk) {
                        uint32_t af[4];
                        const bf* trow = t_s + (mt * 16 + g) * Hp + kk * 16 + 2 * t;
                        af[0] = ld32(trow);
                        af[1] = ld32(trow + 8 * Hp);
                        af[2] = ld32(trow + 8);
                        af[3] = ld32(trow + 8 * Hp + 8);
                        const bf* ph = p_hi + pos_b * Hp + kk * 16 + 2 * t;
                        const bf* pl = p_lo + pos_b * Hp + kk * 16 + 2 * t;
                        mma_16816(cm, af, ld32(ph), ld32(ph + 8));
                        mma_16816(cm, af, ld32(pl), ld32(pl + 8));
                    }
                    // C: rows h = mt * 16 + g (+ 8), columns pos = ntile * 8 + 2t, + 1
                    const int pos_c = ntile * 8 + 2 * t;
                    const int i = pos_c / MM_KEYS, j = pos_c % MM_KEYS;
                    uint32_t hi, lo;
                    split2(cm[0], cm[1], hi, lo);
                    const int at0 = ((mt * 16 + g) * MM_ROWS + i) * ks + j;
                    *reinterpret_cast<uint32_t*>(m_hi + at0) = hi;
                    *reinterpret_cast<uint32_t*>(m_lo + at0) = lo;
                    split2(cm[2], cm[3], hi, lo);
                    const int at1 = ((mt * 16 + g + 8) * MM_ROWS + i) * ks + j;
                    *reinterpret_cast<uint32_t*>(m_hi + at1) = hi;
                    *reinterpret_cast<uint32_t*>(m_lo + at1) = lo;
                }
            }
            __syncthreads();

            // 4. the values
#pragma unroll
            for (int hh = 0; hh < HPW; ++hh) {
                const int h = warp + NW * hh;
                if (h >= H) continue;
                const int c = h / R;
#pragma unroll
                for (int k0 = 0; k0 < MM_KEYS; k0 += 16) {
                    uint32_t ah[4], al[4];
                    const bf* mh = m_hi + (h * MM_ROWS + g) * ks + k0 + 2 * t;
                    const bf* ml = m_lo + (h * MM_ROWS + g) * ks + k0 + 2 * t;
                    ah[0] = ld32(mh); ah[1] = ld32(mh + 8 * ks); ah[2] = ld32(mh + 8); ah[3] = ld32(mh + 8 * ks + 8);
                    al[0] = ld32(ml); al[1] = ld32(ml + 8 * ks); al[2] = ld32(ml + 8); al[3] = ld32(ml + 8 * ks + 8);
#pragma unroll
                    for (int n = 0; n < NV; ++n) {
                        if (n * 8 >= vd) break;
                        const bf* vrow = vt_s + (c * vd + n * 8 + g) * ks + k0 + 2 * t;
                        const uint32_t b0 = ld32(vrow), b1 = ld32(vrow + 8);
                        mma_16816(acc[hh][n], ah, b0, b1);
                        mma_16816(acc[hh][n], al, b0, b1);
                    }
                }
            }
        }
    }

#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        const int h = warp + NW * hh;
        if (h >= H) continue;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            if (!(half ? ok1 : ok0)) continue;
            const int64_t flat = (int64_t)(q_begin + tok0 + g + 8 * half) * H + h;
            if (a.mode == 1) {
                if (t == 0) {
                    const int64_t at = flat * a.num_splits + blockIdx.y;
                    a.part_ml[at * 2] = row_m[hh][half];
                    a.part_ml[at * 2 + 1] = row_l[hh][half];
                }
                continue;
            }
#pragma unroll
            for (int n = 0; n < NV; ++n) {
                if (n * 8 >= vd) break;
                const float x = acc[hh][n][2 * half], y = acc[hh][n][2 * half + 1];
                const int f = n * 8 + 2 * t;
                if (a.mode == 2) {
                    float* dst = a.part_out + (flat * a.num_splits + blockIdx.y) * vd + f;
                    dst[0] = x;
                    dst[1] = y;
                } else {
                    *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<bf*>(a.out) + flat * vd + f) =
                        __floats2bfloat162_rn(x, y);
                }
            }
        }
    }
}

template <int NW, int HPW, int NV>
int launch_mixed_mma(const MixedAttentionArgs& a, int num_seqs, cudaStream_t s) {
    const size_t smem = (size_t)mma_layout(a.n_q, a.n_kv, a.d, a.vd).total;
    static size_t raised = 0;
    if (smem > 48 * 1024 && smem > raised) {
        if (cudaFuncSetAttribute(mixed_head_attention_mma_kernel<NW, HPW, NV>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = smem;
    }
    dim3 grid(num_seqs * a.tiles_per_seq, a.num_splits);
    MB_LAUNCH((mixed_head_attention_mma_kernel<NW, HPW, NV>), grid, NW * 32, smem, s, a);
    return launch_status();
}

// defined in attention_mixed.cu
int launch_mixed_head_sum(const float* part_out, const int* seq_of_token, void* out, int tokens,
                          int n_q, int vd, int num_splits, int dtype, cudaStream_t s);

}  // namespace mb

using namespace mb;

// Whether the tensor-core kernel takes these sizes: heads of a multiple of 16 features, value
// heads of a multiple of 8 up to 128, at most 32 heads (16 when value heads exceed 64), and
// shared memory for a tile's operands.
MB_EXPORT int mb_mixed_head_mma_supports(int n_q, int n_kv, int d, int vd) {
    if (n_q <= 0 || n_kv <= 0 || n_q % n_kv || d <= 0 || d % 16 || d > 256) return 0;
    if (vd <= 0 || vd % 8 || vd > 128) return 0;
    if (n_q > (vd > 64 ? 16 : 32)) return 0;
    return mma_layout(n_q, n_kv, d, vd).total <= 200 * 1024;
}

MB_EXPORT int mb_mixed_head_attention_mma(const void* qkv, int row_width, const void* k_pages,
                                          const void* v_pages, const int* table, int max_pages,
                                          const int* q_start, const int* kv_len, const float* mix,
                                          void* out, int num_seqs, int max_q_len, int n_q, int n_kv,
                                          int d, int vd, int page_size, float scale, int window,
                                          int num_splits, const int* seq_of_token, int tokens,
                                          float* scratch, long long scratch_floats, void* stream) {
    if (num_seqs <= 0 || max_q_len <= 0) return MB_OK;
    if (!mb_mixed_head_mma_supports(n_q, n_kv, d, vd)) return MB_ERR_UNSUPPORTED_SIZE;
    if (page_size <= 0 || (page_size & (page_size - 1))) return MB_ERR_UNSUPPORTED_SIZE;
    if (row_width % 8 || (n_q * d) % 8) return MB_ERR_ALIGNMENT;
    MixedAttentionArgs a;
    a.qkv = qkv; a.row_width = row_width; a.k_pages = k_pages; a.v_pages = v_pages;
    a.table = table; a.max_pages = max_pages; a.q_start = q_start; a.kv_len = kv_len;
    a.mix = mix; a.out = out; a.n_q = n_q; a.n_kv = n_kv; a.d = d; a.vd = vd;
    a.page_size = page_size; a.scale = scale; a.window = window;
    a.bq = MM_ROWS;
    a.tiles_per_seq = (max_q_len + MM_ROWS - 1) / MM_ROWS;
    a.num_splits = 1; a.mode = 0; a.part_ml = a.part_out = nullptr;
    if (num_splits > 1) {
        if (num_splits > 65535 || n_q > 65535) return MB_ERR_UNSUPPORTED_SIZE;
        if (!scratch || scratch_floats < (long long)tokens * n_q * num_splits * (vd + 2)) return MB_ERR_SCRATCH;
        a.num_splits = num_splits;
        a.part_out = scratch;
        a.part_ml = scratch + (int64_t)tokens * n_q * num_splits * vd;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int nv = vd / 8;
    auto run = [&](const MixedAttentionArgs& args) -> int {
#define MB_MM_CASE(NWV, HPWV, NVV) return launch_mixed_mma<NWV, HPWV, NVV>(args, num_seqs, s)
        if (vd <= 64) {
            if (n_q <= 8) { if (nv <= 4) MB_MM_CASE(8, 1, 4); MB_MM_CASE(8, 1, 8); }
            if (n_q <= 16) { if (nv <= 4) MB_MM_CASE(8, 2, 4); MB_MM_CASE(8, 2, 8); }
            if (nv <= 4) MB_MM_CASE(16, 2, 4);
            MB_MM_CASE(16, 2, 8);
        }
        if (n_q <= 8) MB_MM_CASE(8, 1, 16);
        MB_MM_CASE(16, 1, 16);
#undef MB_MM_CASE
    };
    if (num_splits <= 1) return run(a);
    for (int mode = 1; mode <= 2; ++mode) {
        a.mode = mode;
        const int rc = run(a);
        if (rc != MB_OK) return rc;
    }
    return launch_mixed_head_sum(a.part_out, seq_of_token, out, tokens, n_q, vd, num_splits, MB_BF16, s);
}
