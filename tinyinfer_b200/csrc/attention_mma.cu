// bfloat16 paged attention for single decoded tokens, head sizes 64 and 128: a split-KV kernel
// (FlashDecoding: tinyinfer/csrc/flash_decoding.cu:17-336 of the reference, here batched over requests
// in ONE launch, with the query heads of a kv head sharing one read of its keys and values).
//
// Keys and values come straight from the pages: a warp of its own issues TMA tile copies
// (64 keys x 64 features, 128-byte swizzle) into a 3-stage ring guarded by mbarriers; four warps
// consume them with ldmatrix + mma.sync.m16n8k16 (bf16 in, float32 out): a decoded token has at most
// 16 query rows per kv head, far too few for a 128-row tcgen05 tile, and the kernel is bound by HBM,
// not by the tensor pipe. Scores, running maximum (from -inf), sums and outputs are float32;
// probabilities are rounded to bfloat16 for the second product. Masked scores are assigned -inf
// (never added), and value rows that no query of the CTA may see are zeroed in shared memory, so
// stale or unwritten pages cannot leak NaNs.
//
// The split is by position only (256 keys per split), so a request's result does not depend on what
// else is in the batch. Partial results (unnormalised output, maximum, sum per split) go to float32
// scratch and a second kernel merges them. (Prompt portions: attention_prefill_tcgen05.cu.)
#include "sm100_ptx.cuh"

namespace {

constexpr int TK = 64;            // keys per tile
constexpr int CHUNK = 256;        // keys per decode split
constexpr int STAGES = 3;
constexpr int CONSUMER_THREADS = 128;
constexpr int THREADS = CONSUMER_THREADS + 32;

struct AttnParams {
    __nv_bfloat16* out;            // [T, Hq * D]
    const __nv_bfloat16* q;        // [T, Hq, D]
    float* part_o;                 // decode: [rows][Hq][max_splits][D]
    float* part_ml;                // decode: [rows][Hq][max_splits][2]
    const int* rows;               // decode: flat token rows; prefill: tiles as int4 {seq, row0, nrows, pos0}
    const int* positions;
    const int* token_seq;
    const int* block_table;
    int max_blocks, hq, hkv, page_size, num_pages, window, max_splits, num_rows, chunk;
    float scale_log2;              // softmax scale times log2(e)
    int* status;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// Byte offset of (row, 16-byte chunk) inside a tile of 64-feature halves, each [TK][128 B] swizzled.
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * (TK * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

template <int D>
struct Smem {
    static constexpr int HALVES = D / 64;
    static constexpr int TILE_BYTES = HALVES * TK * 128;      // keys OR values of one tile
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int BYTES = 1024 + STAGES * STAGE_BYTES + 128;
    // decode adds its merge buffer: [4 warps][query heads of a kv head <= 16][D + 2] floats
    static int decode_bytes(int group) { return BYTES + 4 * group * (D + 2) * 4; }
};

// Issues the copies of tile `t` (keys t*TK .. t*TK+63 of the request) into a stage. Pieces whose
// page the request does not hold (never written, or given back by a window) are skipped.
template <int D>
__device__ __forceinline__ void load_tile(const CUtensorMap* map, const AttnParams& p, const int* table, int kvh,
                                          int t, uint32_t stage_addr, uint32_t bar) {
    using S = Smem<D>;
    const int piece_rows = p.page_size < TK ? p.page_size : TK;
    const int pieces = TK / piece_rows;
    int pages[4];                                   // page_size >= 16, so at most four pieces
    uint32_t bytes = 0;
    for (int i = 0; i < pieces; ++i) {
        const int tok = t * TK + i * piece_rows;
        const int logical = tok / p.page_size;
        int page = logical < p.max_blocks ? table[logical] : -1;
        if (page >= p.num_pages) page = -1;
        pages[i] = page;
        if (page >= 0) bytes += (uint32_t)piece_rows * 128u * S::HALVES * 2u;
    }
    mbar_expect_tx(bar, bytes);
    for (int i = 0; i < pieces; ++i) {
        if (pages[i] < 0) continue;
        const int tok = t * TK + i * piece_rows;
        const int off = tok % p.page_size;
        const int krow = (pages[i] * p.hkv + kvh) * p.page_size + off;
        const int vrow = ((p.num_pages + pages[i]) * p.hkv + kvh) * p.page_size + off;
#pragma unroll
        for (int hh = 0; hh < S::HALVES; ++hh) {
            const uint32_t dst = stage_addr + hh * (TK * 128) + i * piece_rows * 128;
            tma_load_2d(dst, map, bar, hh * 64, krow);
            tma_load_2d(dst + S::TILE_BYTES, map, bar, hh * 64, vrow);
        }
    }
}

// Zeroes the value rows of a tile outside [keep_lo, keep_hi) (tile-local key indices): no query of
// this CTA may see them and what the stage holds there may be stale or unwritten. Called by the
// `nthreads` threads that will read the tile, `tid` being the caller's index among them.
template <int D>
__device__ __forceinline__ void zero_value_rows(uint8_t* v_tile, int keep_lo, int keep_hi, int tid, int nthreads,
                                                int row_begin, int row_end) {
    constexpr int CHUNKS = D / 8;
    for (int idx = tid; idx < (row_end - row_begin) * CHUNKS; idx += nthreads) {
        const int row = row_begin + idx / CHUNKS, chunk = idx % CHUNKS;
        if (row >= keep_lo && row < keep_hi) continue;
        *reinterpret_cast<uint4*>(v_tile + tile_off(row, chunk)) = make_uint4(0, 0, 0, 0);
    }
}

// ------------------------------------------------------------------------------------ decode
// Persistent: a CTA walks over work items (decode row, kv head, split of 256 keys), item = cta,
// cta + grid, ...; the loading warp runs ahead into the next item while the consumers merge and
// write the current one, so HBM does not idle at item boundaries.
template <int D>
__global__ void __launch_bounds__(THREADS) decode_attention_kernel(const __grid_constant__ CUtensorMap kv_map,
                                                                   const AttnParams p) {
    using S = Smem<D>;
    constexpr int LD = D + 2;                              // merge buffer row: D outputs, maximum, sum
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * S::STAGE_BYTES);
    float* mbuf = reinterpret_cast<float*>(smem + STAGES * S::STAGE_BYTES + 128);   // [4 warps][group][LD]
    const uint32_t bar0 = smem_u32(bars);
    __shared__ int abort_sh;
    volatile int* abort_flag = &abort_sh;

    ti_grid_launch_dependents();
    const int group = p.hq / p.hkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_items = p.num_rows * p.hkv * p.max_splits;
    if (threadIdx.x == 0) {
        abort_sh = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(bar0 + 8u * s, 1); mbar_init(bar0 + 8u * (STAGES + s), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    ti_grid_wait();

    // item -> its row, kv head and key range; false if the split holds no visible key
    struct Item { int r, row, kvh, split, k_begin, k_end; };
    auto get_item = [&](int w, Item& it) {
        it.split = w % p.max_splits;
        const int rest = w / p.max_splits;
        it.kvh = rest % p.hkv;
        it.r = rest / p.hkv;
        it.row = p.rows[it.r];
        const int ctx = p.positions[it.row] + 1;
        const int lo = p.window > 0 ? max(0, ctx - p.window) : 0;
        it.k_begin = max(it.split * p.chunk, lo);
        it.k_end = min(ctx, (it.split + 1) * p.chunk);
        return it.k_begin < it.k_end;
    };

    if (warp == 4) {
        if (lane == 0) {
            uint32_t n = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
                Item it;
                if (!get_item(w, it)) continue;
                const int* table = p.block_table + (size_t)p.token_seq[it.row] * p.max_blocks;
                for (int t = it.k_begin / TK; t < (it.k_end + TK - 1) / TK; ++t, ++n) {
                    const int s = n % STAGES;
                    if (!mbar_wait(bar0 + 8u * (STAGES + s), ((n / STAGES) & 1u) ^ 1u, abort_flag, p.status, 21)) { ok = false; break; }
                    load_tile<D>(&kv_map, p, table, it.kvh, t, smem_u32(smem + s * S::STAGE_BYTES), bar0 + 8u * s);
                }
            }
        }
        return;
    }

    // ---- consumers: the 16 rows of the MMA are the query heads of one kv head (rows >= group are zero)
    const int g = lane >> 2, c = (lane & 3) * 2;
    const int id = lane >> 3, rr = lane & 7;
    uint32_t n = 0;
    for (int w = blockIdx.x; w < num_items; w += gridDim.x) {
        Item item;
        if (!get_item(w, item)) continue;
        uint32_t qa[D / 16][4];
        {
            const __nv_bfloat16* q0 = p.q + ((size_t)item.row * p.hq + (size_t)item.kvh * group) * D;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                qa[ks][0] = g < group ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)g * D + ks * 16 + c) : 0u;
                qa[ks][1] = g + 8 < group ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(g + 8) * D + ks * 16 + c) : 0u;
                qa[ks][2] = g < group ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)g * D + ks * 16 + c + 8) : 0u;
                qa[ks][3] = g + 8 < group ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(g + 8) * D + ks * 16 + c + 8) : 0u;
            }
        }
        float o[D / 8][4];
#pragma unroll
        for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
        const int k_begin = item.k_begin, k_end = item.k_end;

        for (int t = k_begin / TK; t < (k_end + TK - 1) / TK; ++t, ++n) {
            const int s = n % STAGES;
            if (!mbar_wait(bar0 + 8u * s, (n / STAGES) & 1u, abort_flag, p.status, 22)) return;
            uint8_t* k_tile = smem + s * S::STAGE_BYTES;
            uint8_t* v_tile = k_tile + S::TILE_BYTES;
            const int w0 = warp * 16;                         // this warp's 16 keys of the tile
            const int tok0 = t * TK + w0;
            if (tok0 < k_end && tok0 + 16 > k_begin) {
                float sc[2][4] = {};
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t b[4];
                    const int krow = w0 + (id >> 1) * 8 + rr;
                    ldmatrix_x4(b, smem_u32(k_tile) + tile_off(krow, ks * 2 + (id & 1)));
                    mma_bf16(sc[0], qa[ks], b[0], b[1]);
                    mma_bf16(sc[1], qa[ks], b[2], b[3]);
                }
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int tok = tok0 + nb * 8 + c + (j & 1);
                        const float v = (tok >= k_begin && tok < k_end) ? sc[nb][j] * p.scale_log2 : -INFINITY;
                        sc[nb][j] = v;
                        mx[j >> 1] = fmaxf(mx[j >> 1], v);
                    }
                float corr[2], m_use[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                    const float m_new = fmaxf(m_run[h], mx[h]);
                    m_use[h] = m_new == -INFINITY ? 0.f : m_new;
                    corr[h] = exp2f(m_run[h] - m_use[h]);
                    m_run[h] = m_new;
                    l_run[h] *= corr[h];
                }
#pragma unroll
                for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float pv = exp2f(sc[nb][j] - m_use[j >> 1]);
                        sc[nb][j] = pv;
                        l_run[j >> 1] += pv;
                    }
                uint32_t pa[4] = {pack_bf16(sc[0][0], sc[0][1]), pack_bf16(sc[0][2], sc[0][3]),
                                  pack_bf16(sc[1][0], sc[1][1]), pack_bf16(sc[1][2], sc[1][3])};
                if (tok0 < k_begin || tok0 + 16 > k_end) {    // warp-local: only this warp reads these rows
                    zero_value_rows<D>(v_tile, k_begin - t * TK, k_end - t * TK, lane, 32, w0, w0 + 16);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // a later TMA copy overwrites these rows
                    __syncwarp();
                }
#pragma unroll
                for (int nb = 0; nb < D / 8; nb += 2) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        o[nb][j] *= corr[j >> 1];
                        o[nb + 1][j] *= corr[j >> 1];
                    }
                    uint32_t b[4];
                    const int vrow = w0 + (id & 1) * 8 + rr;
                    ldmatrix_x4_trans(b, smem_u32(v_tile) + tile_off(vrow, nb + (id >> 1)));
                    mma_bf16(o[nb], pa, b[0], b[1]);
                    mma_bf16(o[nb + 1], pa, b[2], b[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar0 + 8u * (STAGES + s));
        }

        // ---- merge the four warps (each saw a quarter of the keys) and write the split's partial.
        // Only the rows that are real query heads travel through shared memory.
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");       // the previous item's merge buffer has been read
#pragma unroll
        for (int nb = 0; nb < D / 8; ++nb) {
            float* base = mbuf + ((size_t)warp * group) * LD + nb * 8 + c;
            if (g < group) { base[(size_t)g * LD] = o[nb][0]; base[(size_t)g * LD + 1] = o[nb][1]; }
            if (g + 8 < group) { base[(size_t)(g + 8) * LD] = o[nb][2]; base[(size_t)(g + 8) * LD + 1] = o[nb][3]; }
        }
        if ((lane & 3) == 0) {
            if (g < group) {
                mbuf[((size_t)warp * group + g) * LD + D] = m_run[0];
                mbuf[((size_t)warp * group + g) * LD + D + 1] = l_run[0];
            }
            if (g + 8 < group) {
                mbuf[((size_t)warp * group + g + 8) * LD + D] = m_run[1];
                mbuf[((size_t)warp * group + g + 8) * LD + D + 1] = l_run[1];
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        for (int idx = threadIdx.x; idx < group * D; idx += CONSUMER_THREADS) {
            const int hrow = idx / D, d = idx % D;
            float mw[4], m_all = -INFINITY;
#pragma unroll
            for (int w4 = 0; w4 < 4; ++w4) { mw[w4] = mbuf[((size_t)w4 * group + hrow) * LD + D]; m_all = fmaxf(m_all, mw[w4]); }
            const float m_use = m_all == -INFINITY ? 0.f : m_all;
            float acc = 0.f, l_all = 0.f;
#pragma unroll
            for (int w4 = 0; w4 < 4; ++w4) {
                const float f = exp2f(mw[w4] - m_use);
                acc += f * mbuf[((size_t)w4 * group + hrow) * LD + d];
                l_all += f * mbuf[((size_t)w4 * group + hrow) * LD + D + 1];
            }
            const size_t slot = ((size_t)item.r * p.hq + (size_t)item.kvh * group + hrow) * p.max_splits + item.split;
            p.part_o[slot * D + d] = acc;
            if (d == 0) { p.part_ml[slot * 2] = m_all; p.part_ml[slot * 2 + 1] = l_all; }
        }
    }
}

// One block per (decode row, query head), one thread per feature: merges the splits that hold visible
// keys. The partials of sixteen splits are requested together (one trip to L2 for a context of 4096)
// and folded into a running maximum, sum and output, in split order.
template <int D>
__global__ void decode_merge_kernel(const AttnParams p) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int r = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    const int row = p.rows[r];
    const int ctx = p.positions[row] + 1;
    const int lo = p.window > 0 ? max(0, ctx - p.window) : 0;
    const int s0 = lo / p.chunk;
    int s1 = (ctx - 1) / p.chunk;
    if (s1 >= p.max_splits) {                              // the caller gave fewer splits than the context needs:
        if (d == 0 && p.status) atomicExch(p.status, 23);  // say so, and read nothing that is not this row's
        s1 = p.max_splits - 1;
    }
    const size_t base = ((size_t)r * p.hq + h) * p.max_splits;
    float m_run = -INFINITY, acc = 0.f, l_all = 0.f;
    for (int sb = s0; sb <= s1; sb += 16) {
        float ms[16], ls[16], os[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const bool in = sb + j <= s1;
            const float2 ml = in ? __ldcg(reinterpret_cast<const float2*>(p.part_ml + (base + sb + j) * 2)) : make_float2(-INFINITY, 0.f);
            ms[j] = ml.x;
            ls[j] = ml.y;
            os[j] = in ? __ldcg(p.part_o + (base + sb + j) * D + d) : 0.f;
        }
        float m_new = m_run;
#pragma unroll
        for (int j = 0; j < 16; ++j) m_new = fmaxf(m_new, ms[j]);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float keep = exp2f(m_run - m_use);          // 0 while nothing has been merged yet
        acc *= keep;
        l_all *= keep;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float f = exp2f(ms[j] - m_use);          // 0 for a split that is not there
            acc += f * os[j];
            l_all += f * ls[j];
        }
        m_run = m_new;
    }
    p.out[((size_t)row * p.hq + h) * D + d] = __float2bfloat16_rn(l_all > 0.f ? acc / l_all : 0.f);
}

template <typename K>
int set_smem(K kernel, int bytes, const char* name) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) { ti_set_error("%s: cannot get %d bytes of shared memory: %s", name, bytes, cudaGetErrorString(e)); return (int)e; }
    return 0;
}

int check_shape(int hq, int hkv, int d, int page_size, const char* name) {
    TI_REQUIRE(d == 64 || d == 128, "%s: head_dim %d is not 64 or 128", name, d);
    TI_REQUIRE(hq > 0 && hkv > 0 && hq % hkv == 0 && hq / hkv <= 16, "%s: %d query heads over %d kv heads (at most 16 per kv head)", name, hq, hkv);
    TI_REQUIRE(page_size >= 16 && ((page_size < TK && TK % page_size == 0) || page_size % TK == 0),
               "%s: page size %d must be 16, 32 or a multiple of 64", name, page_size);
    return 0;
}

}  // namespace

// 1 if the tensor-core attention kernels take these sizes.
TI_API int ti_attention_bf16_supported(int hq, int hkv, int d, int page_size) {
    return (d == 64 || d == 128) && hq > 0 && hkv > 0 && hq % hkv == 0 && hq / hkv <= 16 && page_size >= 16 &&
           ((page_size < TK && TK % page_size == 0) || page_size % TK == 0) ? 1 : 0;
}
TI_API int ti_attention_decode_chunk() { return CHUNK; }

namespace {
// Shared memory that decode_attention_kernel<128> (which 0) or <64> (which 1) was last allowed on the
// current device: the attribute is kept per device, so the record is too. nullptr: no current device.
int* configured_bytes(int which) {
    constexpr int MAX_DEVICES = 64;
    static int bytes[2][MAX_DEVICES] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
    return &bytes[which][dev];
}

// CTAs of the decode kernel that run side by side.
int decode_slots(int d, int group) {
    if (d == 128) return ti_sm_count() * (Smem<128>::decode_bytes(group) <= 113 * 1024 ? 2 : 1);
    const int bytes = Smem<64>::decode_bytes(group);
    return ti_sm_count() * (bytes <= 56 * 1024 ? 4 : (bytes <= 75 * 1024 ? 3 : 2));
}
}  // namespace

// Keys per split for a decode step of num_rows requests whose longest context is max_context: 256, or a
// larger power-of-two multiple of it where that is expected to be at least 5 % faster. A work item (row,
// kv head, split) costs about 52 keys' worth of time beyond its keys, the items run in rounds over the
// resident CTAs, and the merge makes one trip to L2 per 16 splits (measured on a B200 at 8 x 4,096 keys:
// 32.1 us with splits of 256, 29.3 with 512; 1 x 32,768: 43.1 and 29.7 with 1,024; with fewer items than
// CTAs the larger split loses, 1 x 4,096: 9.8 and 13.1 us). Smaller splits also even out requests of
// different lengths, hence the margin.
TI_API int ti_attention_decode_plan(int num_rows, int hq, int hkv, int d, int max_context, int window) {
    if (num_rows <= 0 || hkv <= 0 || hq % hkv != 0 || (d != 64 && d != 128)) return CHUNK;
    const int slots = decode_slots(d, hq / hkv);
    const long long visible = window > 0 && window < max_context ? window : max_context;
    int best = CHUNK;
    double best_cost = 0.0;
    for (int c = CHUNK; c <= 8 * CHUNK; c *= 2) {
        const long long splits = (visible + c - 1) / c;
        const long long items = (long long)num_rows * hkv * splits;
        const double cost = (double)((items + slots - 1) / slots) * (c + 52) + (double)((splits + 15) / 16) * 60.0;
        if (c == CHUNK || cost < 0.95 * best_cost) { best = c; best_cost = cost; }
    }
    return best;
}

// Decode: `rows` lists the flat rows of the step whose request brings exactly one token.
// Scratch: part_o float32 [num_rows * hq * max_splits * d], part_ml float32 [num_rows * hq * max_splits * 2];
// chunk: keys per split, a multiple of 256 (ti_attention_decode_plan suggests one); max_splits >=
// ceil(longest context / chunk): a row whose context needs more sets *status to 23 and is computed from
// the keys the splits cover, reading nothing outside its own partials. Calls that share the scratch must
// not overlap.
TI_API int ti_attention_decode_bf16(void* out, const void* q, const void* kv_cache, float* part_o, float* part_ml,
                                    const int* rows, int num_rows, const int* positions, const int* token_seq,
                                    const int* block_table, int max_blocks, int hq, int hkv, int d, int page_size,
                                    int num_pages, float scale, int window, int chunk, int max_splits, int* status,
                                    cudaStream_t stream) {
    if (check_shape(hq, hkv, d, page_size, "attention_decode")) return -1;
    TI_REQUIRE(num_rows >= 0 && num_rows <= 65535 && max_splits > 0 && max_splits <= 65535, "attention_decode: bad sizes");
    TI_REQUIRE(chunk >= CHUNK && chunk % CHUNK == 0, "attention_decode: splits of %d keys are not a multiple of %d", chunk, CHUNK);
    if (num_rows == 0) return 0;
    CUtensorMap map;
    if (!ti_get_bf16_map(kv_cache, 2ll * num_pages * hkv * page_size, d, page_size < TK ? page_size : TK, &map)) return -1;
    AttnParams p;
    p.out = (__nv_bfloat16*)out; p.q = (const __nv_bfloat16*)q; p.part_o = part_o; p.part_ml = part_ml;
    p.rows = rows; p.positions = positions; p.token_seq = token_seq; p.block_table = block_table;
    p.max_blocks = max_blocks; p.hq = hq; p.hkv = hkv; p.page_size = page_size; p.num_pages = num_pages;
    p.chunk = chunk;
    p.window = window; p.max_splits = max_splits; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    p.num_rows = num_rows;
    const int group = hq / hkv;
    const long long items = (long long)num_rows * hkv * max_splits;
    TI_REQUIRE(items < (1ll << 31), "attention_decode: too many work items");
    if (d == 128) {
        const int bytes = Smem<128>::decode_bytes(group);
        int* configured = configured_bytes(0);
        TI_REQUIRE(configured != nullptr, "attention_decode: no current device");
        if (*configured < bytes) { if (set_smem(decode_attention_kernel<128>, bytes, "attention_decode")) return -1; *configured = bytes; }
        const int slots = ti_sm_count() * (bytes <= 113 * 1024 ? 2 : 1);
        ti_launch(decode_attention_kernel<128>, (int)(items < slots ? items : slots), THREADS, bytes, stream, map, p);
        TI_CHECK_LAUNCH("attention_decode");
        ti_launch(decode_merge_kernel<128>, dim3(num_rows, hq), 128, 0, stream, p);
    } else {
        const int bytes = Smem<64>::decode_bytes(group);
        int* configured = configured_bytes(1);
        TI_REQUIRE(configured != nullptr, "attention_decode: no current device");
        if (*configured < bytes) { if (set_smem(decode_attention_kernel<64>, bytes, "attention_decode")) return -1; *configured = bytes; }
        const int slots = ti_sm_count() * (bytes <= 56 * 1024 ? 4 : (bytes <= 75 * 1024 ? 3 : 2));
        ti_launch(decode_attention_kernel<64>, (int)(items < slots ? items : slots), THREADS, bytes, stream, map, p);
        TI_CHECK_LAUNCH("attention_decode");
        ti_launch(decode_merge_kernel<64>, dim3(num_rows, hq), 64, 0, stream, p);
    }
    TI_CHECK_LAUNCH("attention_decode_merge");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// A decode-attention entry point that allocates nothing (declared in tinyinfer_b200_noalloc.h; the
// reference has no counterpart). It is ti_attention_decode_bf16 with the split partials kept in a
// fixed array inside this library instead of a buffer the caller allocates.
//
// Who needs it: code that runs where device allocation is off limits. A plugin called from inside
// another runtime's stream callback or graph-capture region, a serving loop that has handed all free
// memory to its cache and must not grow, or a host that forbids cudaMalloc after start-up for
// latency reasons can still call this: it issues kernel launches only.
//
// The array is `static __device__`: every GPU that loads this library holds TI_NOALLOC_SCRATCH_FLOATS
// floats (8 MB) of it until the process exits. In host code the array's name is only a stand-in, not
// a device address, so the first call on each device looks the address up with
// cudaGetSymbolAddress while that device is current and keeps it; the same call may make the driver
// load this library's code and array onto the device and raises the kernel's shared-memory limit there.
// That first call should be made at start-up, before any stream capture begins and before allocation
// becomes off limits. All calls on a device share the array: two calls that overlap on
// the GPU (different streams, no ordering) race on it. Nothing in it needs clearing between calls:
// every word the merge kernel reads was written by the split kernel of the same call.
constexpr long long TI_NOALLOC_SCRATCH_FLOATS = 2ll * 1024 * 1024;
static __device__ __align__(256) float g_noalloc_decode_scratch[TI_NOALLOC_SCRATCH_FLOATS];

TI_API long long ti_attention_decode_noalloc_capacity() { return TI_NOALLOC_SCRATCH_FLOATS; }

TI_API int ti_attention_decode_bf16_noalloc(void* out, const void* q, const void* kv_cache, const int* rows,
                                            int num_rows, const int* positions, const int* token_seq,
                                            const int* block_table, int max_blocks, int hq, int hkv, int d,
                                            int page_size, int num_pages, float scale, int window, int max_splits,
                                            int* status, cudaStream_t stream) {
    constexpr int MAX_DEVICES = 64;
    static float* scratch_of_device[MAX_DEVICES] = {};
    TI_REQUIRE(num_rows >= 0 && max_splits > 0 && hq > 0 && d > 0, "attention_decode_noalloc: bad sizes");
    const long long need = (long long)num_rows * hq * max_splits * (d + 2);
    TI_REQUIRE(need <= TI_NOALLOC_SCRATCH_FLOATS,
               "attention_decode_noalloc: %d rows x %d heads x %d splits x (%d + 2) = %lld floats exceed the built-in "
               "scratch of %lld floats; use ti_attention_decode_bf16 with a buffer of your own",
               num_rows, hq, max_splits, d, need, TI_NOALLOC_SCRATCH_FLOATS);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    TI_REQUIRE(e == cudaSuccess && dev >= 0 && dev < MAX_DEVICES, "attention_decode_noalloc: no current device (%s)",
               cudaGetErrorString(e));
    if (scratch_of_device[dev] == nullptr) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_decode_scratch);
        TI_REQUIRE(e == cudaSuccess && ptr != nullptr, "attention_decode_noalloc: cudaGetSymbolAddress failed: %s",
                   cudaGetErrorString(e));
        scratch_of_device[dev] = ptr;
    }
    float* part_o = scratch_of_device[dev];
    float* part_ml = part_o + (long long)num_rows * hq * max_splits * d;
    return ti_attention_decode_bf16(out, q, kv_cache, part_o, part_ml, rows, num_rows, positions, token_seq,
                                    block_table, max_blocks, hq, hkv, d, page_size, num_pages, scale, window,
                                    CHUNK, max_splits, status, stream);
}
