// The mixed-head attention of attention_mixed.cu on the tensor cores, for the bfloat16
// engine: scores, the mixing of the heads' weights and the weighted sum of the values are
// all mma.sync products with float32 accumulators.
//
// A block takes 16 query tokens with all their heads and walks the keys twice in tiles of
// 32, as the CUDA-core kernel does (first each row's maximum and sum, then the finished
// weights). Head h belongs to warp h mod (number of warps). Key and value tiles come by
// 16-byte cp.async copies into two buffers, the next tile under way while this one is used.
// Per tile of the second walk:
//   1. S_h = Q_h K^T on the tensor cores (bfloat16 operands are exact, float32 sums),
//      w_h = 2^(S_h * scale * log2 e - max_h) / sum_h in float32 registers;
//   2. every weight is split w = hi + lo into two bfloat16 numbers (|lo| <= 2^-9 |w|, what is
//      left is below 2^-17 |w|) and written to shared memory as [head][token][key];
//   3. the heads are mixed as a product over the head index, W' = M W: M (bfloat16 in the
//      checkpoint, so exact) times hi and times lo, summed in float32. A warp takes tiles
//      of eight (token, key) places, reads every head's weights there (ldmatrix, transposed),
//      and writes the mixed weights, split again, back to the same places;
//   4. O_h += W'_h V on the tensor cores, hi and lo in turn, the value tile read transposed.
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
constexpr int MM_WROW = MM_KEYS + MM_PAD;              // a token's weights: 32 keys + padding
constexpr int MM_WHEAD = MM_ROWS * MM_WROW + MM_PAD;   // a head's weights: 16 tokens + padding

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t ld32(const bf* p) { return *reinterpret_cast<const uint32_t*>(p); }

// Two 8 x 8 tiles of 16-bit elements, transposed: the B operand (k = 16 rows of shared
// memory, n = 8 columns) of one mma from row-major storage. Lanes 0-15 give the rows.
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* smem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
                 : "=r"(r0), "=r"(r1)
                 : "r"(addr));
}

__device__ __forceinline__ void copy_16(void* smem, const void* gmem, bool valid) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zeroed
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(addr), "l"(gmem), "r"(bytes));
}

// 2^x by the special-function unit (relative error about 2^-22); 2^-inf = 0.
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// (x, y) as two pairs of bfloat16: hi = the nearest bfloat16 numbers, lo = what they miss,
// rounded again. One packed conversion per pair; a bfloat16 widens to float32 by a shift.
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(x, y);
    hi = *reinterpret_cast<const uint32_t*>(&h2);
    const float xh = __uint_as_float(hi << 16), yh = __uint_as_float(hi & 0xffff0000u);
    const __nv_bfloat162 l2 = __floats2bfloat162_rn(x - xh, y - yh);
    lo = *reinterpret_cast<const uint32_t*>(&l2);
}

struct MmaLayout {      // offsets in bytes of the shared-memory regions
    int q, k, v, w_hi, w_lo, t, total;
};

__host__ __device__ inline MmaLayout mma_layout(int H, int G, int d, int vd) {
    const int Hp = (H + 15) / 16 * 16;
    MmaLayout l;
    int at = 0;
    l.q = at;     at += H * MM_ROWS * (d + MM_PAD) * 2;
    l.k = at;     at += 2 * G * MM_KEYS * (d + MM_PAD) * 2;       // two buffers
    l.v = at;     at += 2 * G * MM_KEYS * (vd + MM_PAD) * 2;
    l.w_hi = at;  at += Hp * MM_WHEAD * 2;
    l.w_lo = at;  at += Hp * MM_WHEAD * 2;
    l.t = at;     at += Hp * Hp * 2;
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
    bf* v_s = reinterpret_cast<bf*>(smem_raw + L.v);
    bf* w_hi = reinterpret_cast<bf*>(smem_raw + L.w_hi);
    bf* w_lo = reinterpret_cast<bf*>(smem_raw + L.w_lo);
    bf* t_s = reinterpret_cast<bf*>(smem_raw + L.t);
    const int qs = d + MM_PAD, vs = vd + MM_PAD;       // row strides in elements
    const int k_buf = G * MM_KEYS * qs, v_buf = G * MM_KEYS * vs;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int page_shift = __ffs(a.page_size) - 1;

    // queries (zeros for rows beyond the tile), the mixing matrix (identity when absent),
    // zeros in the weights of the heads that pad H to a multiple of 16
    const int chunks = d / 8, vchunks = vd / 8;
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
    for (int idx = tid; idx < (Hp - H) * MM_WHEAD; idx += NW * 32) {
        w_hi[H * MM_WHEAD + idx] = __float2bfloat16_rn(0.f);
        w_lo[H * MM_WHEAD + idx] = __float2bfloat16_rn(0.f);
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

    // A tile's keys (and values) on their way into buffer `buf`; keys beyond the sequence
    // and pages given back arrive as zeros.
    auto issue = [&](int kt, int buf, bool with_values) {
        for (int c = 0; c < G; ++c) {
            for (int e = tid; e < MM_KEYS * chunks; e += NW * 32) {
                const int j = e / chunks, ch = e - j * chunks;
                const int key = kt * MM_KEYS + j;
                int page = -1;
                if (key < kv_len) page = table_page(a.table, seq, a.max_pages, key >> page_shift);
                const bf* src = k_pages;
                if (page >= 0)
                    src += (((int64_t)page * G + c) * a.page_size + (key & (a.page_size - 1))) * d + ch * 8;
                copy_16(k_s + buf * k_buf + (c * MM_KEYS + j) * qs + ch * 8, src, page >= 0);
            }
            if (!with_values) continue;
            for (int e = tid; e < MM_KEYS * vchunks; e += NW * 32) {
                const int j = e / vchunks, ch = e - j * vchunks;
                const int key = kt * MM_KEYS + j;
                int page = -1;
                if (key < kv_len) page = table_page(a.table, seq, a.max_pages, key >> page_shift);
                const bf* src = v_pages;
                if (page >= 0)
                    src += (((int64_t)page * G + c) * a.page_size + (key & (a.page_size - 1))) * vd + ch * 8;
                copy_16(v_s + buf * v_buf + (c * MM_KEYS + j) * vs + ch * 8, src, page >= 0);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    // rows of this thread: g and g + 8 of the tile
    const bool ok0 = g < n_tok, ok1 = g + 8 < n_tok;
    const int pos0 = first_pos + tok0 + g, pos1 = pos0 + 8;
    const float to_log2 = a.scale * 1.4426950408889634f;     // scores in powers of two

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
                    if (ml[2 * z] > -INFINITY) sum += ml[2 * z + 1] * exp2_fast(ml[2 * z] - big);
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
        __syncthreads();       // the pass before is through with both buffers
        if (t_lo < t_hi) issue(t_lo, 0, pass == 1);
        for (int kt = t_lo; kt < t_hi; ++kt) {
            const int buf = (kt - t_lo) & 1;
            asm volatile("cp.async.wait_group 0;\n" ::);
            __syncthreads();   // this tile has arrived for everyone; the tile before is consumed
            if (kt + 1 < t_hi) issue(kt + 1, buf ^ 1, pass == 1);
            const bf* kb = k_s + buf * k_buf;
            const bf* vb = v_s + buf * v_buf;
            // a tile that every row sees whole needs no mask
            const bool whole = kt * MM_KEYS + MM_KEYS - 1 <= p_min && n_tok == MM_ROWS &&
                               (a.window <= 0 || kt * MM_KEYS > p_max - a.window);

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
                const bf* krow = kb + (c * MM_KEYS + g) * qs + 2 * t;
                for (int k0 = 0; k0 < d; k0 += 16) {
                    uint32_t af[4];
                    af[0] = ld32(qrow + k0);
                    af[1] = ld32(qrow + 8 * qs + k0);
                    af[2] = ld32(qrow + k0 + 8);
                    af[3] = ld32(qrow + 8 * qs + k0 + 8);
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
                        mma_16816(s[nt], af, ld32(krow + nt * 8 * qs + k0), ld32(krow + nt * 8 * qs + k0 + 8));
                }
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[nt][e] *= to_log2;
                if (!whole) {
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int key = kt * MM_KEYS + nt * 8 + 2 * t + (e & 1);
                            const int pos = e >= 2 ? pos1 : pos0;
                            bool seen = (e >= 2 ? ok1 : ok0) && key <= pos;
                            if (a.window > 0) seen = seen && key > pos - a.window;
                            if (!seen) s[nt][e] = -INFINITY;
                        }
                }
                if (pass == 0) {
                    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
                        mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
                    }
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                    const float n0 = fmaxf(row_m[hh][0], mx0), n1 = fmaxf(row_m[hh][1], mx1);
                    // a row that has seen nothing yet keeps its maximum at -inf and adds zeros
                    const float b0 = n0 > -INFINITY ? n0 : 0.f, b1 = n1 > -INFINITY ? n1 : 0.f;
                    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        sum0 += exp2_fast(s[nt][0] - b0) + exp2_fast(s[nt][1] - b0);
                        sum1 += exp2_fast(s[nt][2] - b1) + exp2_fast(s[nt][3] - b1);
                    }
                    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
                    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
                    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
                    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
                    row_l[hh][0] = row_l[hh][0] * exp2_fast(row_m[hh][0] - b0) + sum0;
                    row_l[hh][1] = row_l[hh][1] * exp2_fast(row_m[hh][1] - b1) + sum1;
                    row_m[hh][0] = n0;
                    row_m[hh][1] = n1;
                    continue;
                }
                // 2. finished weights, split, [head][token][key]
                const float m0 = row_m[hh][0] > -INFINITY ? row_m[hh][0] : 0.f;
                const float m1 = row_m[hh][1] > -INFINITY ? row_m[hh][1] : 0.f;
                bf* wh = w_hi + h * MM_WHEAD + g * MM_WROW + 2 * t;
                bf* wl = w_lo + h * MM_WHEAD + g * MM_WROW + 2 * t;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    uint32_t hi, lo;
                    split2(exp2_fast(s[nt][0] - m0) * row_l[hh][0], exp2_fast(s[nt][1] - m0) * row_l[hh][0], hi, lo);
                    *reinterpret_cast<uint32_t*>(wh + nt * 8) = hi;
                    *reinterpret_cast<uint32_t*>(wl + nt * 8) = lo;
                    split2(exp2_fast(s[nt][2] - m1) * row_l[hh][1], exp2_fast(s[nt][3] - m1) * row_l[hh][1], hi, lo);
                    *reinterpret_cast<uint32_t*>(wh + 8 * MM_WROW + nt * 8) = hi;
                    *reinterpret_cast<uint32_t*>(wl + 8 * MM_WROW + nt * 8) = lo;
                }
            }
            if (pass == 0) continue;
            __syncthreads();

            // 3. the heads mixed, in place: a warp owns tiles of eight places (token i, keys
            // 8 jb .. 8 jb + 7), reads every head's weights there and writes the mixed ones back
            for (int place = warp; place < MM_ROWS * MM_KEYS / 8; place += NW) {
                const int i = place >> 2, jb = place & 3;
                const int at = i * MM_WROW + jb * 8;
                uint32_t bh[2][2], bl[2][2];
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    if (kk * 16 >= Hp) break;
                    const int head = kk * 16 + (lane & 15);
                    ldmatrix_x2_trans(bh[kk][0], bh[kk][1], w_hi + head * MM_WHEAD + at);
                    ldmatrix_x2_trans(bl[kk][0], bl[kk][1], w_lo + head * MM_WHEAD + at);
                }
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    if (mt * 16 >= Hp) break;
                    float cm[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) {
                        if (kk * 16 >= Hp) break;
                        uint32_t af[4];
                        const bf* trow = t_s + (mt * 16 + g) * Hp + kk * 16 + 2 * t;
                        af[0] = ld32(trow);
                        af[1] = ld32(trow + 8 * Hp);
                        af[2] = ld32(trow + 8);
                        af[3] = ld32(trow + 8 * Hp + 8);
                        mma_16816(cm, af, bh[kk][0], bh[kk][1]);
                        mma_16816(cm, af, bl[kk][0], bl[kk][1]);
                    }
                    // C: rows = heads mt * 16 + g (+ 8), columns = keys 8 jb + 2t, + 1
                    uint32_t hi, lo;
                    split2(cm[0], cm[1], hi, lo);
                    *reinterpret_cast<uint32_t*>(w_hi + (mt * 16 + g) * MM_WHEAD + at + 2 * t) = hi;
                    *reinterpret_cast<uint32_t*>(w_lo + (mt * 16 + g) * MM_WHEAD + at + 2 * t) = lo;
                    split2(cm[2], cm[3], hi, lo);
                    *reinterpret_cast<uint32_t*>(w_hi + (mt * 16 + g + 8) * MM_WHEAD + at + 2 * t) = hi;
                    *reinterpret_cast<uint32_t*>(w_lo + (mt * 16 + g + 8) * MM_WHEAD + at + 2 * t) = lo;
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
                    const bf* mh = w_hi + h * MM_WHEAD + g * MM_WROW + k0 + 2 * t;
                    const bf* ml = w_lo + h * MM_WHEAD + g * MM_WROW + k0 + 2 * t;
                    ah[0] = ld32(mh); ah[1] = ld32(mh + 8 * MM_WROW); ah[2] = ld32(mh + 8); ah[3] = ld32(mh + 8 * MM_WROW + 8);
                    al[0] = ld32(ml); al[1] = ld32(ml + 8 * MM_WROW); al[2] = ld32(ml + 8); al[3] = ld32(ml + 8 * MM_WROW + 8);
                    const bf* vrow = vb + (c * MM_KEYS + k0 + (lane & 15)) * vs;
#pragma unroll
                    for (int n = 0; n < NV; ++n) {
                        if (n * 8 >= vd) break;
                        uint32_t b0, b1;
                        ldmatrix_x2_trans(b0, b1, vrow + n * 8);
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
        // a warp per head while there are at most 16 heads (more warps hide more latency
        // than fewer warps with two heads each), two heads per warp beyond
        if (vd <= 64) {
            if (n_q <= 8) { if (nv <= 4) MB_MM_CASE(8, 1, 4); MB_MM_CASE(8, 1, 8); }
            if (n_q <= 16) { if (nv <= 4) MB_MM_CASE(16, 1, 4); MB_MM_CASE(16, 1, 8); }
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
