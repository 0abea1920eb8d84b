// Attention for one head per work item in one kernel for sm_100a:
//   O[b] = softmax_rows(scale * Q[b] . K[b]^T) . V[b],   f32 storage, TF32 operands, at most 512 keys, V of 32 or 64 columns.
//
// Neither the scores nor the probabilities reach memory.  A CTA computes 128 query rows against all keys of the head
// into tensor memory (the accumulator is the whole row block, up to 512 columns), its epilogue warps turn the scores
// into e = exp(scale * (x - max)) IN PLACE, and a second chain of MMAs multiplies e by V with the A operand read from
// tensor memory (tcgen05.mma with [a_tmem]): the kernel of kernels/attn_softmax.cu, which it follows up to there, then
// has to write 4 n bytes per row and the next matmul has to read them; this one writes 4 dv.
//
//   warp 0 lane 0   producer: Q tile [128 x K] and the key matrix [n x K] as 128-byte-wide K blocks (128-byte swizzle,
//                   rounded to TF32 by the copy engine) through 4-D tensor maps (an operand may be an attention head
//                   split read in place, GemmOperand4D in kernels.h); when the score MMAs have completed, V into the
//                   buffer the keys occupied: either V itself ([n x dv], columns contiguous, possibly a head split
//                   read in place too) as one [keys][128 B] tile per 32 columns, the MN-major B operand, which for
//                   32-bit elements takes the 128-byte swizzle in 32-byte pieces; or V^T ([dv x n], keys contiguous)
//                   as 32-key blocks, the K-major operand with the usual 128-byte swizzle
//   warp 1 lane 0   MMA issuer.  Scores: per half of the keys and K block four tcgen05.mma.kind::tf32 (M 128, N <= 256).
//                   Context: per 32 keys four MMAs (M 128, N dv, K 8) into columns [0, dv) of tensor memory, A = e.
//                   Those columns held the scores of the first dv keys: their e goes through shared memory instead
//                   (a K-major swizzled tile, written by the epilogue warps), so no MMA reads what another overwrites.
//   warps 2..9      epilogue, thread <-> accumulator lane <-> query row, two warps per lane quarter sharing a row's
//                   columns (32 at a time).  Sweep 1: the maximum.  Sweep 2: e, rounded to TF32, over the score (or
//                   into the shared-memory tile), and its sum.  After the context MMAs: O / sum through the warp's
//                   transposing tile into 128-byte lines of the output.
//
// Work items (batch entry, 128-row block) are walked by persistent CTAs.  Every mbarrier wait is bounded as in the
// other tensor-core kernels; the epilogue warps vote before every point where they synchronise with each other.
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

constexpr int kAtThreads = 320;   // producer warp, MMA warp, 8 epilogue warps
constexpr int kAtBlockM = 128;
constexpr int kAtChunkTileBytes = 128 * 128;   // 128 rows x 32 f32: e of one 32-key chunk as an A operand; four warps' transposing tiles
constexpr int kAtStagingBytes = 2 * kAtChunkTileBytes;
constexpr int kAtTraceItems = 16;
constexpr uint32_t kAtSleepNs = 2000;   // the producer and the MMA thread share schedulers with epilogue warps: their waits sleep

struct AttentionParams {
    int32_t n, half_n, halves;       // keys per row; accumulator columns per score MMA (n / halves, at most 256)
    int32_t k_blocks;                // 32-element K blocks of the scores' reduction (the head dimension / 32)
    int32_t dv;                      // columns of V and of the output: 32 or 64
    int32_t m, m_tiles, total;       // rows per batch entry; 128-row blocks per batch entry; work items
    int32_t a_bi, b_bi, v_bi;        // batch entry bt -> map coordinates (bt % bi, bt / bi) of Q, of the keys and of V
    int32_t v_mn;                    // 1: V is given with its columns contiguous ([keys][dv], possibly a head split read in place)
                                     // and is the MN-major B operand of the context MMAs; 0: V^T ([dv][keys]), K-major
    int32_t tmem_cols;
    float scale;
    float* out;                      // [batch][m][dv]: strides out_s0, out_s1 (elements), 1
    int64_t out_s0, out_s1;
    uint32_t* status;
    long long* trace;                // KN_ATTN_TRACE only: 8 clock64 stamps per work item of CTA 0, in pinned host memory
};

__device__ __forceinline__ void at_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__global__ void __launch_bounds__(kAtThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ AttentionParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t q_bytes = (uint32_t)p.k_blocks * (uint32_t)kAtBlockM * 128u;     // [K block][128 rows][128 B]
    const uint32_t k_block_bytes = (uint32_t)p.n * 128u;                             // one K block of the key matrix
    const uint32_t v_block_bytes = (uint32_t)p.dv * 128u;                            // 32 keys of V^T: [dv rows][128 B]
    const uint32_t k_base = base + q_bytes;                                          // keys, then V^T (dv <= K: it fits)
    const uint32_t e_base = k_base + (uint32_t)p.k_blocks * k_block_bytes;           // e of the first dv keys / transposing tiles
    const uint32_t bar_base = e_base + (uint32_t)kAtStagingBytes;
    const uint32_t full_qk = bar_base, s_done = bar_base + 8u, full_v = bar_base + 16u, e_ready = bar_base + 24u;
    const uint32_t pv_done = bar_base + 32u, acc_empty = bar_base + 40u, full_k1 = bar_base + 48u;
    const uint32_t slot_addr = bar_base + 64u;
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + (slot_addr - base));
    volatile int* abandon = (volatile int*)(gen_base + (slot_addr + 4u - base));
    float* exchange_max = (float*)(gen_base + (slot_addr + 16u - base));   // [2 groups][128 rows]: the maximum over a group's columns
    float* exchange_sum = exchange_max + 256;                              // and the sum of their exponentials

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(full_qk, 1);
        mbar_init(full_k1, 1);
        mbar_init(s_done, 1);
        mbar_init(full_v, 1);
        mbar_init(e_ready, 256);
        mbar_init(pv_done, 1);
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
    const int chunks = p.n >> 5;          // 32-key chunks of a row
    const int e_chunks = p.dv >> 5;       // of which the first go through shared memory
    asm volatile("griddepcontrol.wait;" ::: "memory");   // nothing above touches global memory

    if (warp == 0 && lane == 0) {
        // ---------------- producer
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
        // (the second half of the keys, if the score MMAs take them in two halves, has a barrier of its own: the MMAs over
        // the first half run while it lands)
        const uint32_t half_bytes = (uint32_t)p.k_blocks * (uint32_t)p.half_n * 128u;
        const uint32_t qk_bytes = q_bytes + half_bytes;
        const uint32_t v_bytes = (uint32_t)chunks * v_block_bytes;
        // Q of an item is requested a phase ahead of its keys: its buffer is free once the previous item's score MMAs
        // have read it, the keys' only when that item's context MMAs have read V.  One barrier takes both.
        auto request_q = [&](int item) {
            const int ibt = item / p.m_tiles, imt = item - ibt * p.m_tiles;
            mbar_expect_tx(full_qk, qk_bytes);
            for (int kb = 0; kb < p.k_blocks; kb++)
                tma_load_4d(base + (uint32_t)kb * (uint32_t)kAtBlockM * 128u, &map_q, full_qk, kb * 32, imt * kAtBlockM, ibt % p.a_bi, ibt / p.a_bi);
        };
        if ((int)blockIdx.x < p.total) request_q((int)blockIdx.x);
        int local = 0;
        for (int t = blockIdx.x; t < p.total; t += gridDim.x, local++) {
            const int bt = t / p.m_tiles;
            // the context MMAs of the previous item have read V
            if (local > 0 && !mbar_wait(pv_done, (uint32_t)((local - 1) & 1), abandon, p.status, 41, kWaitCycles, kAtSleepNs)) break;
            if (p.trace && blockIdx.x == 0 && local < kAtTraceItems) p.trace[local * 8 + 0] = clock64();
            const int b2 = bt % p.b_bi, b3 = bt / p.b_bi;
            if (p.halves > 1) mbar_expect_tx(full_k1, half_bytes);
            for (int h = 0; h < p.halves; h++)
                for (int kb = 0; kb < p.k_blocks; kb++)
                    tma_load_4d(k_base + (uint32_t)kb * k_block_bytes + (uint32_t)(h * p.half_n) * 128u, &map_k, h == 0 ? full_qk : full_k1,
                                kb * 32, h * p.half_n, b2, b3);
            // the score MMAs have read the keys: V^T takes their place while the epilogue works on the scores
            if (!mbar_wait(s_done, (uint32_t)(local & 1), abandon, p.status, 42, kWaitCycles, kAtSleepNs)) break;
            mbar_expect_tx(full_v, v_bytes);
            if (p.v_mn) {
                // per 32 columns of V a tile [keys][128 B] (at most 256 rows per request)
                const int v2 = bt % p.v_bi, v3 = bt / p.v_bi;
                const int rows_per = p.n > 256 ? p.n >> 1 : p.n;
                for (int cb = 0; cb < e_chunks; cb++)
                    for (int r0 = 0; r0 < p.n; r0 += rows_per)
                        tma_load_4d(k_base + (uint32_t)(cb * p.n + r0) * 128u, &map_v, full_v, cb * 32, r0, v2, v3);
            } else {
                for (int c = 0; c < chunks; c++) tma_load_4d(k_base + (uint32_t)c * v_block_bytes, &map_v, full_v, c * 32, 0, bt, 0);
            }
            if (t + (int)gridDim.x < p.total) request_q(t + (int)gridDim.x);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer: f32 accumulate, TF32 x TF32, both K-major, M = 128
        const uint32_t idesc_s = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.half_n >> 3) << 17) | ((uint32_t)(kAtBlockM >> 4) << 24);
        // (bit 16: the B operand is MN-major, its N index contiguous)
        const uint32_t idesc_o = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.v_mn ? 1 : 0) << 16) | ((uint32_t)(p.dv >> 3) << 17) |
                                 ((uint32_t)(kAtBlockM >> 4) << 24);
        // MN-major B of 32-bit elements: the 128-byte swizzle in 32-byte pieces (layout type 1; the copy engine's
        // SWIZZLE_128B_ATOM_32B).  4 K rows (keys) of 128 bytes (32 columns of V) make an atom, the next 4 keys are
        // `stride byte offset` = 512 bytes further on, the next 32 columns `leading byte offset` (their own
        // [keys][128 B] tile).
        const uint64_t v_mn_desc = ((uint64_t)(((uint32_t)p.n * 128u) >> 4) << 16) | ((uint64_t)(512 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)1 << 61);
        int local = 0;
        for (int t = blockIdx.x; t < p.total; t += gridDim.x, local++) {
            if (!mbar_wait(full_qk, (uint32_t)(local & 1), abandon, p.status, 43, kWaitCycles, kAtSleepNs)) break;
            if (p.trace && blockIdx.x == 0 && local < kAtTraceItems) p.trace[local * 8 + 1] = clock64();
            // the epilogue has read the previous item's output from tensor memory
            if (local > 0 && !mbar_wait(acc_empty, (uint32_t)((local - 1) & 1), abandon, p.status, 44, kWaitCycles, kAtSleepNs)) break;
            tc_fence_after();
            if (p.trace && blockIdx.x == 0 && local < kAtTraceItems) p.trace[local * 8 + 2] = clock64();
            if (t + (int)gridDim.x >= p.total) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            bool landed = true;
            for (int h = 0; h < p.halves && landed; h++) {
                if (h == 1) {
                    landed = mbar_wait(full_k1, (uint32_t)(local & 1), abandon, p.status, 43, kWaitCycles, kAtSleepNs);
                    if (!landed) break;
                    tc_fence_after();
                }
                const uint32_t acc = tmem_base + (uint32_t)(h * p.half_n);
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    const uint64_t da = smem_desc_sw128(base + (uint32_t)kb * (uint32_t)kAtBlockM * 128u);
                    const uint64_t db = smem_desc_sw128(k_base + (uint32_t)kb * k_block_bytes + (uint32_t)(h * p.half_n) * 128u);
#pragma unroll
                    for (int j = 0; j < 4; j++) mma_tf32(acc, da + 2u * j, db + 2u * j, idesc_s, (kb | j) != 0 ? 1u : 0u);
                }
            }
            if (!landed) break;
            mma_commit(s_done);
            // context: O[128 x dv] = e[128 x n] . V[n x dv]
            if (!mbar_wait(full_v, (uint32_t)(local & 1), abandon, p.status, 45, kWaitCycles, kAtSleepNs)) break;
            if (!mbar_wait(e_ready, (uint32_t)(local & 1), abandon, p.status, 46, kWaitCycles, kAtSleepNs)) break;
            tc_fence_after();
            for (int c = 0; c < chunks; c++) {
                // B of the j-th instruction of the chunk (8 keys): K-major, 32 bytes along the rows of the chunk's block
                // of V^T; MN-major, 8 rows of 128 bytes further on in the tiles of V
                const uint64_t db = p.v_mn ? (v_mn_desc | (uint64_t)(((k_base + (uint32_t)c * 4096u) & 0x3FFFFu) >> 4))
                                           : smem_desc_sw128(k_base + (uint32_t)c * v_block_bytes);
                const uint32_t db_step = p.v_mn ? (1024u >> 4) : 2u;
                if (c < e_chunks) {
                    const uint64_t da = smem_desc_sw128(e_base + (uint32_t)c * kAtChunkTileBytes);
#pragma unroll
                    for (int j = 0; j < 4; j++) mma_tf32(tmem_base, da + 2u * j, db + db_step * j, idesc_o, (c | j) != 0 ? 1u : 0u);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++) mma_tf32_a_tmem(tmem_base, tmem_base + (uint32_t)(c * 32 + j * 8), db + db_step * j, idesc_o, 1u);
                }
            }
            mma_commit(pv_done);
        }
    } else if (warp >= 2) {
        // ---------------- epilogue
        // Two groups of four warps (one warp per lane quarter each): group g takes the 32-column chunks g, g + 2, ...
        // of every row; the two groups exchange their rows' maximum and sum.
        const int quarter = warp & 3;
        const int group = (warp - 2) >> 2;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        const uint32_t row_phase = (uint32_t)row_in_tile & 7u;
        // the output goes through the warp's own 4 KB tile (its rows of chunk tile `group`): a thread writes 32 columns
        // of its row (16-byte pieces, XOR-swizzled by the row: no bank conflicts on either side), then eight lanes read
        // a row's 128 bytes back and store them as one line
        const uint32_t warp_tile = e_base + (uint32_t)group * kAtChunkTileBytes + (uint32_t)(quarter * 32) * 128u;
        const int read_row = lane >> 3;                       // + 4 i for the i-th of eight reads
        const uint32_t read_piece = (uint32_t)lane & 7u;
        // The warps synchronise with each other (named barriers), so they must agree on going on after every wait
        // that can give up: one lane waits, then all vote.
        auto wait_agreed = [&](uint32_t bar, uint32_t parity, uint32_t code) -> bool {
            uint32_t good = 1;
            if (lane == 0) good = mbar_wait(bar, parity, abandon, p.status, code, kWaitCycles, kAtSleepNs) ? 1u : 0u;
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
            if (!all_good) return false;
            while (!mbar_try_wait(bar, parity)) {}
            return true;
        };
        int local = 0;
        for (int t = blockIdx.x; t < p.total; t += gridDim.x, local++) {
            const int bt = t / p.m_tiles, mt = t - bt * p.m_tiles;
            const bool trace = p.trace && blockIdx.x == 0 && local < kAtTraceItems && lane == 0 && quarter == 2 && group == 0;
            if (!wait_agreed(s_done, (uint32_t)(local & 1), 47)) break;
            tc_fence_after();
            if (trace) p.trace[local * 8 + 3] = clock64();
            // The sweeps are software-pipelined: the tensor-memory load of the next chunk is in flight while this one
            // is worked on (`tcgen05.wait::ld` waits for every outstanding load, so it comes right before the next issue).
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
            exchange_max[group * 128 + row_in_tile] = mx;
            asm volatile("bar.sync 3, 256;" ::: "memory");
            mx = fmaxf(mx, exchange_max[(group ^ 1) * 128 + row_in_tile]);
            if (trace) p.trace[local * 8 + 4] = clock64();
            // sweep 2: e = 2^(x * scale * log2(e) - max * scale * log2(e)) and its sum; e rounded to TF32 (the tensor
            // cores drop the low 13 bits: half of the last kept place is added first) replaces the score as the A operand
            const float scale2 = p.scale * 1.4426950408889634f;
            const float neg_max2 = -mx * scale2;
            float sum = 0.f;
            auto sweep_exp = [&](int c, uint32_t (&v)[32]) {
                float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float e0 = exp2_approx(fmaf(__uint_as_float(v[j]), scale2, neg_max2));
                    const float e1 = exp2_approx(fmaf(__uint_as_float(v[j + 1]), scale2, neg_max2));
                    const float e2 = exp2_approx(fmaf(__uint_as_float(v[j + 2]), scale2, neg_max2));
                    const float e3 = exp2_approx(fmaf(__uint_as_float(v[j + 3]), scale2, neg_max2));
                    v[j] = __float_as_uint(e0) + 0x1000u, v[j + 1] = __float_as_uint(e1) + 0x1000u;
                    v[j + 2] = __float_as_uint(e2) + 0x1000u, v[j + 3] = __float_as_uint(e3) + 0x1000u;
                    s0 += e0, s1 += e1, s2 += e2, s3 += e3;
                }
                sum += (s0 + s1) + (s2 + s3);
                if (c < e_chunks) {
                    const uint32_t row_addr = e_base + (uint32_t)c * kAtChunkTileBytes + (uint32_t)row_in_tile * 128u;
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (((uint32_t)q ^ row_phase) << 4)), "r"(v[4 * q]),
                                     "r"(v[4 * q + 1]), "r"(v[4 * q + 2]), "r"(v[4 * q + 3])
                                     : "memory");
                } else {
                    tmem_store_32(row_tmem + (uint32_t)(c * 32), v);
                }
            };
            if (group < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)(group * 32), va);
#pragma unroll 1
            for (int c = group; c < chunks; c += 4) {
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c + 2 < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)((c + 2) * 32), vb);
                sweep_exp(c, va);
                if (c + 2 >= chunks) break;
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c + 4 < chunks) tmem_load_32_nowait(row_tmem + (uint32_t)((c + 4) * 32), va);
                sweep_exp(c + 2, vb);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the shared-memory tile is read by the tensor cores
            tc_fence_before();
            at_mbar_arrive(e_ready);
            if (trace) p.trace[local * 8 + 5] = clock64();
            // the sums meet while the context MMAs run
            exchange_sum[group * 128 + row_in_tile] = sum;
            asm volatile("bar.sync 3, 256;" ::: "memory");
            // (Each table is rewritten for the next item only after the other barrier of that item, which a group
            // reaches after its reads of this item's.)
            sum += exchange_sum[(group ^ 1) * 128 + row_in_tile];
            const float inv = 1.0f / sum;
            if (!wait_agreed(pv_done, (uint32_t)(local & 1), 48)) break;
            tc_fence_after();
            if (trace) p.trace[local * 8 + 6] = clock64();
            // the output: group g takes columns [32 g, 32 g + 32)
            if (group < e_chunks) {
                tmem_load_32(row_tmem + (uint32_t)(group * 32), va);
#pragma unroll
                for (int j = 0; j < 32; j++) va[j] = __float_as_uint(__uint_as_float(va[j]) * inv);
                const uint32_t tile_write = warp_tile + (uint32_t)lane * 128u;
#pragma unroll
                for (int q = 0; q < 8; q++)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile_write + (((uint32_t)q ^ ((uint32_t)lane & 7u)) << 4)),
                                 "r"(va[4 * q]), "r"(va[4 * q + 1]), "r"(va[4 * q + 2]), "r"(va[4 * q + 3])
                                 : "memory");
                __syncwarp();
                const int rows_left = p.m - mt * kAtBlockM - quarter * 32;   // rows of this warp inside the matrix
                float* dst = p.out + (int64_t)bt * p.out_s0 + (int64_t)(mt * kAtBlockM + quarter * 32 + read_row) * p.out_s1 +
                             (int64_t)(group * 32) + (int64_t)(read_piece * 4u);
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
                __syncwarp();
            }
            if (trace) p.trace[local * 8 + 7] = clock64();
            // every tcgen05.ld of this item has completed: the MMA thread may overwrite tensor memory
            tc_fence_before();
            at_mbar_arrive(acc_empty);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
    }
}

struct AttentionLaunch {
    CUtensorMap map_q, map_k, map_v;
    AttentionParams p;
    dim3 grid;
    int smem_bytes;
};

}  // namespace

bool attention_fits(int64_t batch, int64_t m, int64_t n, int64_t k, int64_t dv) {
    if (!attn_softmax_fits(batch, m, n, k)) return false;
    if (!(dv == 32 || dv == 64) || dv > k) return false;
    const int64_t smem = 1024 + (kAtBlockM + n) * k * 4 + kAtStagingBytes + 2560;
    return smem <= 227 * 1024;
}

std::shared_ptr<void> attention_prepare(const GemmParams& g, uint32_t* status_word) {
    if (g.half || g.conv_operand != 0 || g.splits > 1 || g.add1 || g.add2 || g.act != 0 || g.row_softmax != 2 || !g.values) return nullptr;
    if (!attention_fits(g.batch, g.m, g.n, g.k, g.values_cols)) return nullptr;
    if (g.sc[2] != 1 || g.sc[1] % 4 != 0 || (g.batch > 1 && g.sc[0] % 4 != 0) || ((uintptr_t)g.c & 15) != 0) return nullptr;
    // V^T [batch][dv][n] with the keys contiguous, or (values_mn) V [batch][n][dv] with its columns contiguous / a head split
    if (((uintptr_t)g.values & 15) != 0) return nullptr;
    if (!g.v4.enabled && (g.values_strides[2] != 1 || g.values_strides[1] % 4 != 0 ||
                          (g.batch > 1 && (g.values_strides[0] % 4 != 0 || g.values_strides[0] == 0))))
        return nullptr;
    if (g.v4.enabled && (!g.values_mn || g.v4.kd != g.values_cols || g.v4.rd < g.n || g.v4.strides[0] != 1)) return nullptr;
    auto l = std::make_shared<AttentionLaunch>();
    AttentionParams& p = l->p;
    memset(&p, 0, sizeof(p));
    p.n = (int)g.n;
    p.halves = g.n > 256 ? 2 : 1;
    p.half_n = p.n / p.halves;
    p.k_blocks = (int)(g.k / 32);
    p.dv = (int)g.values_cols;
    p.m = (int)g.m;
    p.m_tiles = (int)((g.m + kAtBlockM - 1) / kAtBlockM);
    const int64_t total = (int64_t)p.m_tiles * g.batch;
    if (total > (1 << 30)) return nullptr;
    p.total = (int)total;
    p.scale = g.softmax_scale;
    p.status = status_word;
    p.out = (float*)g.c;
    p.out_s0 = g.sc[0], p.out_s1 = g.sc[1];
    p.tmem_cols = 32;
    while (p.tmem_cols < std::max(p.n, p.dv)) p.tmem_cols <<= 1;
    // Q and the keys through 4-D maps (K offset, row, x, y): a head split read in place as it is (its K offset is not
    // split), a plain [batch, rows, K] operand with x = the batch entry (bi = batch + 1: coordinates (bt, 0))
    {
        int box[4] = {32, kAtBlockM, 1, 1};
        if (g.a4.enabled) {
            if (g.a4.kd != g.k || g.a4.rd < g.m || g.a4.strides[0] != 1) return nullptr;
            l->map_q = tc_make_map(g.a, 4, g.a4.dims, g.a4.strides, box, true);
            p.a_bi = g.a4.bi;
        } else {
            if (g.batch > 1 && g.sa[0] == 0) return nullptr;
            int64_t dims[4] = {g.k, g.m, g.batch, 1}, strides[4] = {1, g.sa[1], g.sa[0], 4};
            l->map_q = tc_make_map(g.a, 4, dims, strides, box, true);
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
    p.v_mn = g.values_mn ? 1 : 0;
    if (g.values_mn) {
        int box[4] = {32, (int)(g.n > 256 ? g.n / 2 : g.n), 1, 1};
        if (g.v4.enabled) {
            l->map_v = tc_make_map_mn_major(g.values, 4, g.v4.dims, g.v4.strides, box);
            p.v_bi = g.v4.bi;
        } else {
            int64_t dims[4] = {g.values_cols, g.n, g.batch, 1}, strides[4] = {1, g.values_strides[1], g.batch > 1 ? g.values_strides[0] : g.values_strides[1] * g.n, 4};
            l->map_v = tc_make_map_mn_major(g.values, 4, dims, strides, box);
            p.v_bi = (int)g.batch + 1;
        }
    } else {
        int box[4] = {32, p.dv, 1, 1};
        int64_t dims[4] = {g.n, g.values_cols, g.batch, 1}, strides[4] = {1, g.values_strides[1], g.batch > 1 ? g.values_strides[0] : g.values_strides[1] * g.values_cols, 4};
        l->map_v = tc_make_map(g.values, 4, dims, strides, box, true);
        p.v_bi = (int)g.batch + 1;
    }
    // KN_ATTN_TRACE=1 in the environment: CTA 0 stamps clock64 per work item (producer: loads issued; MMA thread:
    // operands landed, tensor memory free; first epilogue warp: scores ready, after the maximum, after the
    // exponentials, context ready, output stored) and the table is printed when the process exits.  A measuring aid.
    if (getenv("KN_ATTN_TRACE")) {
        static long long* table = nullptr;
        if (!table && cudaHostAlloc((void**)&table, (size_t)kAtTraceItems * 64, cudaHostAllocMapped) == cudaSuccess) {
            memset(table, 0, (size_t)kAtTraceItems * 64);
            atexit([] {
                const long long* d = table;
                fprintf(stderr, "attention_kernel, CTA 0, SM clock cycles since the item's loads were issued\n"
                                "item  operands_landed  tensor_memory_free  scores_ready  maximum  exponentials  context_ready  output_stored  item_period\n");
                for (int i = 0; i < kAtTraceItems && d[i * 8 + 7]; i++) {
                    fprintf(stderr, "%4d", i);
                    for (int j = 1; j < 8; j++) fprintf(stderr, "  %12lld", d[i * 8 + j] - d[i * 8]);
                    fprintf(stderr, "  %12lld\n", i ? d[i * 8] - d[(i - 1) * 8] : 0);
                }
            });
        }
        p.trace = table;
    }
    l->smem_bytes = 1024 + (int)((kAtBlockM + g.n) * g.k * 4) + kAtStagingBytes + 2560;   // (+ barriers, control words, the exchange tables)
    l->grid = dim3((unsigned)std::min<int64_t>(total, 148), 1, 1);
    return l;
}

int attention_launch(const void* launch, cudaStream_t stream) {
    const AttentionLaunch& l = *(const AttentionLaunch*)launch;
    static std::mutex mu;
    static bool done[64] = {false};
    int device = 0;
    cudaGetDevice(&device);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (device >= 0 && device < 64 && !done[device]) {
            cudaError_t e = cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return (int)e;
            done[device] = true;
        }
    }
    launch_pdl(attention_kernel, dim3(l.grid), dim3(kAtThreads), (size_t)(l.smem_bytes), stream, l.map_q, l.map_k, l.map_v, l.p);
    return (int)cudaGetLastError();
}

}  // namespace kn
