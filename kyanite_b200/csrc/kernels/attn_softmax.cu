// Attention scores and their softmax in one kernel for sm_100a:  P[b] = softmax_rows(scale * Q[b] . K[b]^T),
// f32 storage, TF32 operands, rows of at most 512 keys.
//
// Planned step by step the scores are written (one HBM pass), read and written again by the softmax (two more) and
// read by the next matmul: with a reduction as short as a head (K = 64) those passes are all the time there is.
// Here a CTA computes 128 query rows against ALL keys of a head into tensor memory (the accumulator is the whole
// row block: up to 512 columns), and its epilogue warps turn the rows into probabilities on the way out: the scores
// never reach memory.
//
//   warp 0 lane 0   producer: the Q tile [128 x K] and the K matrix [keys x K] of the work item, as 128-byte-wide K
//                   blocks (128-byte swizzle, rounded to TF32 by the copy engine), through 4-D tensor maps: an
//                   operand may be an attention head split read in place (GemmOperand4D, kernels.h)
//   warp 1 lane 0   MMA issuer: per half of the keys (at most 256 accumulator columns per instruction) and K block,
//                   four tcgen05.mma.kind::tf32; tcgen05.commit frees the operand buffer and signals the accumulator
//   warps 2..9      epilogue, thread <-> accumulator lane <-> query row, two warps per lane quarter sharing a row's
//                   columns.  Three sweeps over the row in tensor memory, 32 columns at a time: the maximum; then
//                   e = exp(scale * (x - max)) written back over the score (tcgen05.st) and the sum of e; then
//                   e / sum through the warp's transposing tile into 128-byte lines of the output.  One exponential and
//                   about six instructions per element: with the exponential in both of two sweeps and the
//                   denormal fix-ups of expf the warps issued 20 per element and the kernel took twice as long.
//
// Work items (batch entry, 128-row block) are walked by persistent CTAs.  The operand buffer is single (K alone is up
// to 128 KB): the next item's loads start when this item's MMAs have completed and run under its epilogue, which is
// the long part.  Every mbarrier wait is bounded as in the other tensor-core kernels.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>

#include "../tc.h"
#include "tc_host.h"
#include "tc_ptx.cuh"
#include "launch.cuh"

namespace kn {

namespace {

using namespace tcp;

constexpr int kAsThreads = 320;   // producer warp, MMA warp, 8 epilogue warps
constexpr int kAsBlockM = 128;
constexpr int kAsWarpTileBytes = 32 * 128;     // an epilogue warp's transposing tile: 32 rows x 32 f32 columns
constexpr int kAsStagingBytes = 8 * kAsWarpTileBytes;

struct AttnSoftmaxParams {
    int32_t n, half_n, halves;       // keys per row; accumulator columns per MMA (n / halves, at most 256)
    int32_t k_blocks;                // 32-element K blocks (the head dimension / 32)
    int32_t m_tiles, total;          // 128-row blocks per batch entry; work items
    int32_t a_bi, b_bi;              // batch entry bt -> map coordinates (bt % bi, bt / bi) of each operand
    int32_t tmem_cols;
    int32_t m;                       // rows per batch entry (the last row block of an entry may be partial)
    float* out;                      // probabilities [batch][m][n]: strides out_s0, out_s1 (elements), 1
    int64_t out_s0, out_s1;
    float scale;
    uint32_t* status;
    long long* trace;                // KN_ATTN_TRACE only: 8 clock64 stamps per work item of CTA 0, in pinned host memory
};
constexpr int kAsTraceItems = 16;

__device__ __forceinline__ void as_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__global__ void __launch_bounds__(kAsThreads, 1)
attn_softmax_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ AttnSoftmaxParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t q_bytes = (uint32_t)p.k_blocks * (uint32_t)kAsBlockM * 128u;     // [K block][128 rows][128 B]
    const uint32_t k_block_bytes = (uint32_t)p.n * 128u;                             // one K block of the key matrix
    const uint32_t k_base = base + q_bytes;
    const uint32_t staging_base = k_base + (uint32_t)p.k_blocks * k_block_bytes;     // one transposing tile per epilogue warp
    const uint32_t bar_base = staging_base + (uint32_t)kAsStagingBytes;
    const uint32_t full_bar = bar_base, free_bar = bar_base + 8u, acc_full = bar_base + 16u, acc_empty = bar_base + 24u;
    const uint32_t slot_addr = bar_base + 32u;
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + (slot_addr - base));
    volatile int* abandon = (volatile int*)(gen_base + (slot_addr + 4u - base));
    float* exchange_max = (float*)(gen_base + (slot_addr + 16u - base));   // [2 groups][128 rows]: the maximum over a group's columns
    float* exchange_sum = exchange_max + 256;                              // and the sum of their exponentials

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(full_bar, 1);
        mbar_init(free_bar, 1);
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 256);
        *abandon = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"((uint32_t)p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    asm volatile("griddepcontrol.wait;" ::: "memory");   // nothing above touches global memory

    if (warp == 0 && lane == 0) {
        // ---------------- producer
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        const uint32_t bytes = q_bytes + (uint32_t)p.k_blocks * k_block_bytes;
        int local = 0;
        for (int t = blockIdx.x; t < p.total; t += gridDim.x, local++) {
            const int bt = t / p.m_tiles, mt = t - bt * p.m_tiles;
            // the MMAs of the previous item have read the operand buffer
            if (local > 0 && !mbar_wait(free_bar, (uint32_t)((local - 1) & 1), abandon, p.status, 31)) break;
            if (p.trace && blockIdx.x == 0 && local < kAsTraceItems) p.trace[local * 8 + 0] = clock64();
            mbar_expect_tx(full_bar, bytes);
            const int a2 = bt % p.a_bi, a3 = bt / p.a_bi, b2 = bt % p.b_bi, b3 = bt / p.b_bi;
            for (int kb = 0; kb < p.k_blocks; kb++) {
                tma_load_4d(base + (uint32_t)kb * (uint32_t)kAsBlockM * 128u, &map_q, full_bar, kb * 32, mt * kAsBlockM, a2, a3);
                for (int h = 0; h < p.halves; h++)
                    tma_load_4d(k_base + (uint32_t)kb * k_block_bytes + (uint32_t)(h * p.half_n) * 128u, &map_k, full_bar, kb * 32,
                                h * p.half_n, b2, b3);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer: f32 accumulate, TF32 x TF32, both K-major, M = 128, N = half_n
        const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.half_n >> 3) << 17) | ((uint32_t)(kAsBlockM >> 4) << 24);
        int local = 0;
        for (int t = blockIdx.x; t < p.total; t += gridDim.x, local++) {
            if (!mbar_wait(full_bar, (uint32_t)(local & 1), abandon, p.status, 32)) break;
            if (p.trace && blockIdx.x == 0 && local < kAsTraceItems) p.trace[local * 8 + 1] = clock64();
            // the epilogue has read the previous item's accumulator
            if (local > 0 && !mbar_wait(acc_empty, (uint32_t)((local - 1) & 1), abandon, p.status, 33)) break;
            tc_fence_after();
            if (p.trace && blockIdx.x == 0 && local < kAsTraceItems) p.trace[local * 8 + 2] = clock64();
            if (t + (int)gridDim.x >= p.total) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            for (int h = 0; h < p.halves; h++) {
                const uint32_t acc = tmem_base + (uint32_t)(h * p.half_n);
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    const uint64_t da = smem_desc_sw128(base + (uint32_t)kb * (uint32_t)kAsBlockM * 128u);
                    const uint64_t db = smem_desc_sw128(k_base + (uint32_t)kb * k_block_bytes + (uint32_t)(h * p.half_n) * 128u);
#pragma unroll
                    for (int j = 0; j < 4; j++) mma_tf32(acc, da + 2u * j, db + 2u * j, idesc, (kb | j) != 0 ? 1u : 0u);
                }
            }
            mma_commit(free_bar);
            mma_commit(acc_full);
        }
    } else if (warp >= 2) {
        // ---------------- epilogue
        // Two groups of four warps (one warp per lane quarter each): group g takes the 32-column chunks g, g + 2, ...
        // of every row; the two groups exchange their rows' maximum and sum between the sweeps.  With one warp per row quarter
        // (one warp per scheduler) the exponentials of a 512-key row bound the kernel.
        const int quarter = warp & 3;
        const int group = (warp - 2) >> 2;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        const int chunks = p.n >> 5;
        // sweep 3 goes through the warp's own tile: a thread writes 32 columns of its row (16-byte pieces, XOR-swizzled
        // by the row so that neither side has bank conflicts), then eight lanes read a row's 128 bytes back and
        // store them as one line
        const uint32_t warp_tile = staging_base + (uint32_t)(warp - 2) * kAsWarpTileBytes;
        const uint32_t tile_write = warp_tile + (uint32_t)lane * 128u;
        const uint32_t write_phase = (uint32_t)lane & 7u;
        const int read_row = lane >> 3;                       // + 4 i for the i-th of eight reads
        const uint32_t read_piece = (uint32_t)lane & 7u;
        int local = 0;
        for (int t = blockIdx.x; t < p.total; t += gridDim.x, local++) {
            const int bt = t / p.m_tiles, mt = t - bt * p.m_tiles;
            const bool trace = p.trace && blockIdx.x == 0 && local < kAsTraceItems && lane == 0 && quarter == 2;
            {
                // the four warps synchronise with each other below, so they must agree on going on: vote
                uint32_t good = 1;
                if (lane == 0) good = mbar_wait(acc_full, (uint32_t)(local & 1), abandon, p.status, 34) ? 1u : 0u;
                good = __shfl_sync(0xffffffffu, good, 0);
                uint32_t all_good;
                asm volatile(
                    "{\n\t.reg .pred p, q;\n\t"
                    "setp.ne.u32 p, %1, 0;\n\t"
                    "bar.red.and.pred q, 4, 256, p;\n\t"
                    "selp.u32 %0, 1, 0, q;\n\t}"
                    : "=r"(all_good)
                    : "r"(good)
                    : "memory");
                if (!all_good) break;
                while (!mbar_try_wait(acc_full, (uint32_t)(local & 1))) {}
            }
            tc_fence_after();
            if (trace && group == 0) p.trace[local * 8 + 3] = clock64();
            // Three sweeps over the row's columns in tensor memory, 32 at a time, each software-pipelined (the load of
            // the next chunk is in flight while this one is worked on; `tcgen05.wait::ld` waits for every outstanding
            // load, so it comes right before the next issue).  One exponential per element: the second sweep writes
            // exp(x - max) back over the score, the third only scales.
            uint32_t va[32], vb[32];
            const uint32_t row_tmem = tmem_base + lane_bits;
            // sweep 1: the maximum of the raw scores (the scale is positive: the planner checks)
            float mx = -INFINITY;
            auto sweep_max = [&](const uint32_t (&v)[32]) {
                float m0 = mx, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    m0 = fmaxf(m0, __uint_as_float(v[j]));
                    m1 = fmaxf(m1, __uint_as_float(v[j + 1]));
                    m2 = fmaxf(m2, __uint_as_float(v[j + 2]));
                    m3 = fmaxf(m3, __uint_as_float(v[j + 3]));
                }
                mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            };
            if (group < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)(group * 32), va);
#pragma unroll 1
            for (int c = group; c < chunks; c += 4) {
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c + 2 < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)((c + 2) * 32), vb);
                sweep_max(va);
                if (c + 2 >= chunks) break;
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c + 4 < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)((c + 4) * 32), va);
                sweep_max(vb);
            }
            // the other group's columns of the row
            exchange_max[group * 128 + row_in_tile] = mx;
            asm volatile("bar.sync 3, 256;" ::: "memory");
            mx = fmaxf(mx, exchange_max[(group ^ 1) * 128 + row_in_tile]);
            if (trace && group == 0) p.trace[local * 8 + 4] = clock64();
            // sweep 2: e = 2^(x * scale * log2(e) - max * scale * log2(e)) over the score, and the sum of e
            const float scale2 = p.scale * 1.4426950408889634f;
            const float neg_max2 = -mx * scale2;
            float sum = 0.f;
            auto sweep_exp = [&](uint32_t taddr, uint32_t (&v)[32]) {
                float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float e0 = exp2_approx(fmaf(__uint_as_float(v[j]), scale2, neg_max2));
                    const float e1 = exp2_approx(fmaf(__uint_as_float(v[j + 1]), scale2, neg_max2));
                    const float e2 = exp2_approx(fmaf(__uint_as_float(v[j + 2]), scale2, neg_max2));
                    const float e3 = exp2_approx(fmaf(__uint_as_float(v[j + 3]), scale2, neg_max2));
                    v[j] = __float_as_uint(e0), v[j + 1] = __float_as_uint(e1);
                    v[j + 2] = __float_as_uint(e2), v[j + 3] = __float_as_uint(e3);
                    s0 += e0, s1 += e1, s2 += e2, s3 += e3;
                }
                sum += (s0 + s1) + (s2 + s3);
                tmem_store_32(taddr, v);
            };
            if (group < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)(group * 32), va);
#pragma unroll 1
            for (int c = group; c < chunks; c += 4) {
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c + 2 < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)((c + 2) * 32), vb);
                sweep_exp(row_tmem + (uint32_t)(c * 32), va);
                if (c + 2 >= chunks) break;
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c + 4 < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)((c + 4) * 32), va);
                sweep_exp(row_tmem + (uint32_t)((c + 2) * 32), vb);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            exchange_sum[group * 128 + row_in_tile] = sum;
            asm volatile("bar.sync 3, 256;" ::: "memory");
            // (Each table is rewritten for the next item only after the other barrier of that item, which a group
            // reaches after its reads of this item's.)
            sum += exchange_sum[(group ^ 1) * 128 + row_in_tile];
            const float inv = 1.0f / sum;
            if (trace && group == 0) p.trace[local * 8 + 5] = clock64();
            // sweep 3: the probabilities, written as full 128-byte lines with plain stores.  (Bulk tensor stores of
            // 128-row x 32-column tiles from staging tiles measured 26 bytes per clock per SM however few CTAs ran,
            // a store holds its tile for over a thousand cycles: this sweep took half of the item's time.)
            const int rows_left = p.m - mt * kAsBlockM - quarter * 32;   // rows of this warp inside the matrix
            float* const out_warp = p.out + (int64_t)bt * p.out_s0 + (int64_t)(mt * kAsBlockM + quarter * 32 + read_row) * p.out_s1 +
                                    (int64_t)(read_piece * 4u);
            auto sweep_store = [&](int c, uint32_t (&v)[32]) {
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) * inv);
                __syncwarp();   // the reads of the previous chunk
#pragma unroll
                for (int q = 0; q < 8; q++)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile_write + (((uint32_t)q ^ write_phase) << 4)), "r"(v[4 * q]),
                                 "r"(v[4 * q + 1]), "r"(v[4 * q + 2]), "r"(v[4 * q + 3])
                                 : "memory");
                __syncwarp();
                float* dst = out_warp + c * 32;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int row = 4 * i + read_row;
                    uint32_t x0, x1, x2, x3;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3)
                                 : "r"(warp_tile + (uint32_t)row * 128u + ((read_piece ^ ((uint32_t)row & 7u)) << 4))
                                 : "memory");
                    if (row < rows_left)
                        asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(dst + (int64_t)(4 * i) * p.out_s1), "r"(x0), "r"(x1), "r"(x2), "r"(x3)
                                     : "memory");
                }
            };
            if (group < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)(group * 32), va);
#pragma unroll 1
            for (int c = group; c < chunks; c += 4) {
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c + 2 < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)((c + 2) * 32), vb);
                sweep_store(c, va);
                if (c + 2 >= chunks) break;
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c + 4 < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)((c + 4) * 32), va);
                sweep_store(c + 2, vb);
            }
            if (trace) p.trace[local * 8 + 6 + group] = clock64();
            // every tcgen05.ld of this accumulator has completed: the MMA thread may overwrite it
            tc_fence_before();
            as_mbar_arrive(acc_empty);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
    }
}

struct AttnSoftmaxLaunch {
    CUtensorMap map_q, map_k;
    AttnSoftmaxParams p;
    dim3 grid;
    int smem_bytes;
};

}  // namespace

bool attn_softmax_fits(int64_t batch, int64_t m, int64_t n, int64_t k) {
    if (batch < 1 || batch > (1 << 24) || m < 128 || n < 32 || n > 512 || n % 32 != 0 || k < 32 || k % 32 != 0) return false;
    const int64_t halves = n > 256 ? 2 : 1;
    if ((n / halves) % 16 != 0) return false;
    const int64_t smem = 1024 + (kAsBlockM + n) * k * 4 + kAsStagingBytes + 2560;
    return smem <= 227 * 1024;
}

std::shared_ptr<void> attn_softmax_prepare(const GemmParams& g, uint32_t* status_word) {
    if (g.half || g.conv_operand != 0 || g.splits > 1 || g.add1 || g.add2 || g.act != 0) return nullptr;
    if (!attn_softmax_fits(g.batch, g.m, g.n, g.k)) return nullptr;
    if (g.sc[2] != 1 || g.sc[1] % 4 != 0 || (g.batch > 1 && g.sc[0] % 4 != 0) || ((uintptr_t)g.c & 15) != 0) return nullptr;
    auto l = std::make_shared<AttnSoftmaxLaunch>();
    AttnSoftmaxParams& p = l->p;
    memset(&p, 0, sizeof(p));
    p.n = (int)g.n;
    p.halves = g.n > 256 ? 2 : 1;
    p.half_n = p.n / p.halves;
    p.k_blocks = (int)(g.k / 32);
    p.m_tiles = (int)((g.m + kAsBlockM - 1) / kAsBlockM);
    const int64_t total = (int64_t)p.m_tiles * g.batch;
    if (total > (1 << 30)) return nullptr;
    p.total = (int)total;
    p.scale = g.softmax_scale;
    p.status = status_word;
    p.tmem_cols = 32;
    while (p.tmem_cols < p.n) p.tmem_cols <<= 1;
    // both operands through 4-D maps (K offset, row, x, y): a head split read in place as it is (its K offset is not
    // split), a plain [batch, rows, K] operand with x = the batch entry (bi = batch + 1: coordinates (bt, 0))
    {
        int box[4] = {32, kAsBlockM, 1, 1};
        if (g.a4.enabled) {
            if (g.a4.kd != g.k || g.a4.rd < g.m || g.a4.strides[0] != 1) return nullptr;
            l->map_q = tc_make_map(g.a, 4, g.a4.dims, g.a4.strides, box, true);
            p.a_bi = g.a4.bi;
        } else {
            const bool shared = g.batch > 1 && g.sa[0] == 0;
            int64_t dims[4] = {g.k, g.m, shared ? 1 : g.batch, 1}, strides[4] = {1, g.sa[1], shared ? 4 : g.sa[0], 4};
            l->map_q = tc_make_map(g.a, 4, dims, strides, box, true);
            if (shared) return nullptr;   // (no caller needs it: every batch entry has its own queries)
            p.a_bi = (int)g.batch + 1;
        }
    }
    {
        int box[4] = {32, p.half_n, 1, 1};
        if (g.b4.enabled) {
            if (g.b4.kd != g.k || g.b4.rd < g.n || g.b4.strides[0] != 1) return nullptr;
            l->map_k = tc_make_map(g.b, 4, g.b4.dims, g.b4.strides, box, true);
            p.b_bi = g.b4.bi;
        } else {
            if (g.batch > 1 && g.sb[0] == 0) return nullptr;
            int64_t dims[4] = {g.k, g.n, g.batch, 1}, strides[4] = {1, g.sb[2], g.sb[0], 4};
            l->map_k = tc_make_map(g.b, 4, dims, strides, box, true);
            p.b_bi = (int)g.batch + 1;
        }
    }
    p.m = (int)g.m;
    p.out = (float*)g.c;
    p.out_s0 = g.sc[0], p.out_s1 = g.sc[1];
    const int operands = 1024 + (int)((kAsBlockM + g.n) * g.k * 4) + 2560;   // (+ barriers, control words, the exchange table)
    // KN_ATTN_TRACE=1 in the environment: CTA 0 stamps clock64 per work item (producer: loads issued; MMA thread:
    // operands landed, accumulator free; first epilogue warp of each group: accumulator ready, end of each sweep) and
    // the table is printed when the process exits.  A measuring aid.
    if (getenv("KN_ATTN_TRACE")) {
        static long long* table = nullptr;
        if (!table && cudaHostAlloc((void**)&table, (size_t)kAsTraceItems * 64, cudaHostAllocMapped) == cudaSuccess) {
            memset(table, 0, (size_t)kAsTraceItems * 64);
            atexit([] {
                const long long* d = table;
                fprintf(stderr, "attn_softmax_kernel, CTA 0, SM clock cycles since the item's loads were issued\n"
                                "item  operands_landed  accumulator_free  accumulator_ready  maximum  exponentials  stores_group0  stores_group1  item_period\n");
                for (int i = 0; i < kAsTraceItems && d[i * 8 + 6]; i++) {
                    fprintf(stderr, "%4d", i);
                    for (int j = 1; j < 8; j++) fprintf(stderr, "  %12lld", d[i * 8 + j] - d[i * 8]);
                    fprintf(stderr, "  %12lld\n", i ? d[i * 8] - d[(i - 1) * 8] : 0);
                }
            });
        }
        p.trace = table;
    }
    l->smem_bytes = operands + kAsStagingBytes;
    l->grid = dim3((unsigned)std::min<int64_t>(total, 148), 1, 1);
    // KN_ATTN_GRID=<n> in the environment: at most n CTAs (measuring: how the store sweep depends on how many SMs store)
    if (const char* e = getenv("KN_ATTN_GRID")) l->grid.x = (unsigned)std::max(1, std::min(atoi(e), (int)l->grid.x));
    return l;
}

int attn_softmax_launch(const void* launch, cudaStream_t stream) {
    const AttnSoftmaxLaunch& l = *(const AttnSoftmaxLaunch*)launch;
    static std::mutex mu;
    static bool done[64] = {false};
    int device = 0;
    cudaGetDevice(&device);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (device >= 0 && device < 64 && !done[device]) {
            cudaError_t e = cudaFuncSetAttribute(attn_softmax_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return (int)e;
            done[device] = true;
        }
    }
    launch_pdl(attn_softmax_kernel, dim3(l.grid), dim3(kAsThreads), (size_t)(l.smem_bytes), stream, l.map_q, l.map_k, l.p);
    return (int)cudaGetLastError();
}

}  // namespace kn
