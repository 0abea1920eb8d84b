// Tensor-core contractions for sm_100a: batched matrix multiply and stride-1 2D convolution as an
// implicit GEMM, TF32 operands, f32 accumulation in tensor memory, fused epilogue
// act(acc + add1 + add2).
//
// One CTA computes one 128 x BN output tile:
//   warp 0 / lane 0   TMA producer: per K block one `cp.async.bulk.tensor` for the 128 x 32 A tile and
//                     one for the BN x 32 B tile, both K-major with the 128-byte swizzle, into a
//                     ring of shared-memory stages guarded by full/empty mbarriers
//   warp 1 / lane 0   MMA issuer: four `tcgen05.mma.kind::tf32` (K = 8 each) per stage into a
//                     128-lane x BN-column f32 accumulator in TMEM; `tcgen05.commit` frees the stage
//   warps 2..5        epilogue: `tcgen05.ld` the accumulator (one output row per thread), add the
//                     optional addends, activation, store through the output's element strides
//
// Convolution needs no im2col buffer: the input is read as a 4-D (C, W, H, N) tensor, an M tile is
// a box of nb x hb x wb output positions, and filter tap (r, s) is the same box shifted by
// (r - pad_y, s - pad_x); positions outside the image are zero-filled by the TMA unit, which is
// exactly the zero padding of the convolution.  Channel and K tails are zero-filled the same way.
//
// Every mbarrier wait is bounded: on expiry the kernel records a code in the executor's status word,
// all roles leave their loops, TMEM is released and the kernel returns.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../tc.h"
#include "tc_host.h"
#include "tc_ptx.cuh"
#include "epilogue.cuh"
#include "launch.cuh"

namespace kn {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockK = 32;                     // floats: one 128-byte swizzle row
constexpr int kATileBytes = kBlockM * 128;
constexpr int kThreads = 192;

struct TcParams {
    int32_t mode;   // 0 = matmul, 1 = conv
    int32_t bn, tmem_cols, k_iters, stages;
    int32_t splits, k_iters_total;   // matmul split K: slices per batch entry, K blocks overall (k_iters = per slice)
    int32_t a_batch, b_batch;        // matmul: 1, or 0 when every batch entry uses the same A / B (batch stride 0)
    // conv tiling
    int32_t cblocks, kernel_w, pad_y, pad_x, wb, hb, nb, tiles_w, tiles_h;
    int32_t wb_shift, hb_shift;   // log2 of wb, hb
    int32_t n_img, oh, ow;
    int64_t m, n;           // matmul rows / columns (conv: n = output channels)
    float* out;
    const float* add1;
    const float* add2;
    int64_t so[4], s1[4], s2[4];   // conv: (n, c, h, w) strides; matmul: (batch, row, col, -)
    int32_t act, round_tf32;
    int32_t staged;         // epilogue goes through shared memory (output columns are unit-stride)
    int32_t vec4;           // staged epilogue may use 128-bit accesses
    int32_t add1_mode, add2_mode;   // vec4 path: 0 absent, 1 one value per column (bias), 2 full tensor
    uint32_t* status;
};

using namespace tcp;   // PTX wrappers (kernels/tc_ptx.cuh)

__device__ __forceinline__ float finish(float v, int act, int round_tf32) {
    v = apply_activation(v, act);
    if (round_tf32) {
        uint32_t u;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
        v = __uint_as_float(u);
    }
    return v;
}

// ---------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(kThreads, 1)
tc_contract_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int stages = p.stages;
    const uint32_t b_tile_bytes = (uint32_t)p.bn * 128u;
    const uint32_t a_base = base;
    const uint32_t b_base = base + (uint32_t)stages * kATileBytes;
    // The barriers and control words sit behind whichever is larger, the operand stages or the tile the
    // staged epilogue transposes through (128 rows of bn + 4 floats, which reuses the stages' memory): with
    // few stages and a wide tile the staging tile is the larger one and must not reach the barriers, which
    // other epilogue warps may still be polling.
    const uint32_t operand_end = b_base + (uint32_t)stages * b_tile_bytes;
    const uint32_t staging_end = base + (p.staged ? (uint32_t)kBlockM * (uint32_t)(p.bn + 4) * 4u : 0u);
    const uint32_t bar_base = operand_end > staging_end ? operand_end : staging_end;   // 8-byte aligned
    const uint32_t full_bar = bar_base, empty_bar = bar_base + 8u * stages, accum_bar = bar_base + 16u * stages;
    const uint32_t slot_addr = accum_bar + 8u;
    // generic pointers to the same words
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + (slot_addr - base));
    volatile int* abandon = (volatile int*)(gen_base + (slot_addr + 4u - base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(full_bar + 8u * s, 1);
            mbar_init(empty_bar + 8u * s, 1);
        }
        mbar_init(accum_bar, 1);
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
    pdl_enter();   // nothing above touches global memory

    // tile coordinates
    int m0 = 0, n0_img = 0, h0 = 0, w0 = 0;
    const int ncol0 = blockIdx.y * p.bn;
    // matmul with split K: blockIdx.z enumerates (batch, K slice); each slice writes its own partial tile
    const int zb = blockIdx.z;
    const int batch = p.mode == 0 ? zb / p.splits : 0;
    const int k_first = p.mode == 0 ? (zb - batch * p.splits) * p.k_iters : 0;   // first K block of this slice
    const int k_count = p.mode == 0 ? min(p.k_iters, p.k_iters_total - k_first) : p.k_iters;
    if (p.mode == 0) {
        m0 = blockIdx.x * kBlockM;
    } else {
        const int tw = blockIdx.x % p.tiles_w;
        const int th = (blockIdx.x / p.tiles_w) % p.tiles_h;
        const int tn = blockIdx.x / (p.tiles_w * p.tiles_h);
        w0 = tw * p.wb;
        h0 = th * p.hb;
        n0_img = tn * p.nb;
    }

    if (warp == 0 && lane == 0) {
        // ---------------- producer
        for (int it = 0; it < k_count; it++) {
            const int s = it % stages;
            const uint32_t parity = ((it / stages) & 1) ^ 1;
            if (!mbar_wait(empty_bar + 8u * s, parity, abandon, p.status, 1)) break;
            mbar_expect_tx(full_bar + 8u * s, kATileBytes + b_tile_bytes);
            if (p.mode == 0) {
                tma_load_4d(a_base + s * kATileBytes, &map_a, full_bar + 8u * s, (k_first + it) * kBlockK, m0, batch * p.a_batch, 0);
                tma_load_3d(b_base + s * b_tile_bytes, &map_b, full_bar + 8u * s, (k_first + it) * kBlockK, ncol0, batch * p.b_batch);
            } else {
                const int tap = it / p.cblocks, cb = it - tap * p.cblocks;
                const int r = tap / p.kernel_w, sx = tap - r * p.kernel_w;
                tma_load_4d(a_base + s * kATileBytes, &map_a, full_bar + 8u * s, cb * kBlockK, w0 + sx - p.pad_x,
                            h0 + r - p.pad_y, n0_img);
                tma_load_3d(b_base + s * b_tile_bytes, &map_b, full_bar + 8u * s, cb * kBlockK, ncol0, tap);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        // instruction descriptor: f32 accumulate, tf32 x tf32, both K-major, M = 128, N = bn
        const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(kBlockM >> 4) << 24);
        bool ok = true;
        for (int it = 0; it < k_count && ok; it++) {
            const int s = it % stages;
            const uint32_t parity = (it / stages) & 1;
            ok = mbar_wait(full_bar + 8u * s, parity, abandon, p.status, 2);
            if (!ok) break;
            tc_fence_after();
            const uint64_t da = smem_desc_sw128(a_base + s * kATileBytes);
            const uint64_t db = smem_desc_sw128(b_base + s * b_tile_bytes);
#pragma unroll
            for (int j = 0; j < kBlockK / 8; j++)   // 8 tf32 = 32 bytes per instruction: advance the start address by 2 units
                mma_tf32(tmem_base, da + 2u * j, db + 2u * j, idesc, (it | j) != 0 ? 1u : 0u);
            mma_commit(empty_bar + 8u * s);
        }
        if (ok) mma_commit(accum_bar);
    } else if (warp >= 2) {
        // ---------------- epilogue: thread <-> accumulator lane <-> output row
        const int q = warp & 3;
        const bool ok = mbar_wait(accum_bar, 0, abandon, p.status, 3);
        tc_fence_after();
        const int64_t sn_o = p.mode == 0 ? p.so[2] : p.so[1];
        const int64_t sn_1 = p.mode == 0 ? p.s1[2] : p.s1[1];
        const int64_t sn_2 = p.mode == 0 ? p.s2[2] : p.s2[1];
        // offsets of output row `row` of this tile in the output and the two addends
        auto row_offsets = [&](int row, int64_t& off_o, int64_t& off_1, int64_t& off_2) -> bool {
            if (p.mode == 0) {
                const int64_t m = (int64_t)m0 + row;
                off_o = zb * p.so[0] + m * p.so[1];   // (with split K the output is the slice's partial tile)
                off_1 = batch * p.s1[0] + m * p.s1[1];
                off_2 = batch * p.s2[0] + m * p.s2[1];
                return m < p.m;
            }
            // wb and hb are powers of two: no integer division on this path
            const int wi = row & (p.wb - 1);
            const int hi = (row >> p.wb_shift) & (p.hb - 1);
            const int ni = row >> (p.wb_shift + p.hb_shift);
            const int64_t img = n0_img + ni, oy = h0 + hi, ox = w0 + wi;
            off_o = img * p.so[0] + oy * p.so[2] + ox * p.so[3];
            off_1 = img * p.s1[0] + oy * p.s1[2] + ox * p.s1[3];
            off_2 = img * p.s2[0] + oy * p.s2[2] + ox * p.s2[3];
            return img < p.n_img && oy < p.oh && ox < p.ow;
        };
        if (ok && !p.staged) {
            // Output rows are the unit-stride direction (e.g. NCHW): the 32 lanes of a warp hold 32
            // consecutive rows, so storing straight from registers is already coalesced.
            int64_t off_o, off_1, off_2;
            const bool row_valid = row_offsets(q * 32 + lane, off_o, off_1, off_2);
            for (int c0 = 0; c0 < p.bn; c0 += 32) {
                uint32_t v[32];
                tmem_load_32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                if (!row_valid) continue;
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int64_t n = (int64_t)ncol0 + c0 + j;
                    if (c0 + j < p.bn && n < p.n) {
                        float acc = __uint_as_float(v[j]);
                        if (p.add1) acc += p.add1[off_1 + n * sn_1];
                        if (p.add2) acc += p.add2[off_2 + n * sn_2];
                        p.out[off_o + n * sn_o] = finish(acc, p.act, p.round_tf32);
                    }
                }
            }
        } else if (ok) {
            // Output columns are the unit-stride direction (channels-last, row-major C): transpose
            // through shared memory (the operand stages are all consumed by now) so that a warp
            // writes one output row's consecutive columns per instruction.
            float* tile = (float*)gen_base;
            const int ld = p.bn + 4;
            const int row = q * 32 + lane;
            for (int c0 = 0; c0 < p.bn; c0 += 32) {
                uint32_t v[32];
                tmem_load_32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    if (c0 + j < p.bn)
                        *(float4*)(tile + row * ld + c0 + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                           __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                }
            }
            __syncwarp();   // each warp reads back only the 32 rows it staged itself
            if (p.vec4) {
                // 128-bit path: a lane owns four consecutive columns; eight rows are in flight at a
                // time so the addend loads overlap instead of serialising on memory latency
                for (int c = 4 * lane; c < p.bn; c += 128) {
                    const int64_t n = (int64_t)ncol0 + c;
                    if (n >= p.n) continue;
                    float4 col_add = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (p.add1_mode == 1) col_add = *(const float4*)(p.add1 + n);
                    if (p.add2_mode == 1) {
                        const float4 t = *(const float4*)(p.add2 + n);
                        col_add.x += t.x; col_add.y += t.y; col_add.z += t.z; col_add.w += t.w;
                    }
#pragma unroll 1
                    for (int rr = 0; rr < 32; rr += 8) {
                        float4 extra[8];
                        int64_t off_out[8];
                        bool valid[8];
#pragma unroll
                        for (int u = 0; u < 8; u++) {
                            int64_t off_1, off_2;
                            valid[u] = row_offsets(q * 32 + rr + u, off_out[u], off_1, off_2);
                            extra[u] = col_add;
                            if (valid[u] && p.add1_mode == 2) {
                                const float4 t = *(const float4*)(p.add1 + off_1 + n);
                                extra[u].x += t.x; extra[u].y += t.y; extra[u].z += t.z; extra[u].w += t.w;
                            }
                            if (valid[u] && p.add2_mode == 2) {
                                const float4 t = *(const float4*)(p.add2 + off_2 + n);
                                extra[u].x += t.x; extra[u].y += t.y; extra[u].z += t.z; extra[u].w += t.w;
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 8; u++) {
                            if (!valid[u]) continue;
                            const float4 a = *(const float4*)(tile + (q * 32 + rr + u) * ld + c);
                            float4 o;
                            o.x = finish(a.x + extra[u].x, p.act, p.round_tf32);
                            o.y = finish(a.y + extra[u].y, p.act, p.round_tf32);
                            o.z = finish(a.z + extra[u].z, p.act, p.round_tf32);
                            o.w = finish(a.w + extra[u].w, p.act, p.round_tf32);
                            *(float4*)(p.out + off_out[u] + n) = o;
                        }
                    }
                }
            } else {
                for (int r = q * 32; r < q * 32 + 32; r++) {
                    int64_t off_o, off_1, off_2;
                    if (!row_offsets(r, off_o, off_1, off_2)) continue;
                    for (int c = lane; c < p.bn; c += 32) {
                        const int64_t n = (int64_t)ncol0 + c;
                        if (n < p.n) {
                            float acc = tile[r * ld + c];
                            if (p.add1) acc += p.add1[off_1 + n * sn_1];
                            if (p.add2) acc += p.add2[off_2 + n * sn_2];
                            p.out[off_o + n * sn_o] = finish(acc, p.act, p.round_tf32);
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------- split-K reduction
// Sums the per-slice partial tiles [batch][slice][M][N] of a split-K matmul and applies the epilogue.
struct SplitKReduceParams {
    const float* partial;
    int32_t splits;
    int64_t batch, m, n;
    float* out;
    const float* add1;
    const float* add2;
    int64_t so[3], s1[3], s2[3];
    int32_t act, round_tf32;
    int32_t half;   // out and the addends hold f16 elements (the partial sums are always f32)
};

__global__ void __launch_bounds__(256) splitk_reduce_kernel(const __grid_constant__ SplitKReduceParams p) {
    pdl_enter();
    const int64_t total = p.batch * p.m * p.n;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
        const int64_t n = idx % p.n;
        const int64_t m = (idx / p.n) % p.m;
        const int64_t b = idx / (p.n * p.m);
        const float* src = p.partial + (b * p.splits * p.m + m) * p.n + n;
        float acc = 0.f;
        for (int s = 0; s < p.splits; s++) acc += src[(int64_t)s * p.m * p.n];
        if (p.half) {
            if (p.add1) acc += __half2float(((const __half*)p.add1)[b * p.s1[0] + m * p.s1[1] + n * p.s1[2]]);
            if (p.add2) acc += __half2float(((const __half*)p.add2)[b * p.s2[0] + m * p.s2[1] + n * p.s2[2]]);
            ((__half*)p.out)[b * p.so[0] + m * p.so[1] + n * p.so[2]] = __float2half_rn(apply_activation(acc, p.act));
            continue;
        }
        if (p.add1) acc += p.add1[b * p.s1[0] + m * p.s1[1] + n * p.s1[2]];
        if (p.add2) acc += p.add2[b * p.s2[0] + m * p.s2[1] + n * p.s2[2]];
        p.out[b * p.so[0] + m * p.so[1] + n * p.so[2]] = finish(acc, p.act, p.round_tf32);
    }
}

// ---------------------------------------------------------------- channels-last convolution kernel
//
// Same pipeline, operands swapped: the accumulator holds output channels on its 128 lanes and
// output pixels on its columns, D[k][pixel] = sum_{r,s,c} W[k][c][r][s] * X[pixel + (r, s)][c].
//   A operand  the filter: for one horizontal tap s and one block of 32 input channels, the R
//              vertical taps arrive as R tiles of [128 output channels x 32] in ONE bulk copy
//   B operand  the activations: a sub-tile is hb rows x 8 columns of one image; its input window
//              for horizontal tap s, (hb + R - 1) rows x 8 pixels x 32 channels, is loaded ONCE and
//              vertical tap r reads it at a row offset of r * 1024 bytes (8 pixels x 128 bytes),
//              which keeps every operand descriptor 1024-byte aligned
// so the activations cross from L2 S times instead of R*S times, and a CTA that owns `per_cta`
// sub-tiles loads the filter once for all of them.  (An SM pulls a bounded number of bytes per
// clock from L2; at TF32 that, not the tensor pipe, limits a 128x128 tile that re-fetches both
// operands per tap.)
//
// With channels-last output a warp's 32 lanes are 32 consecutive channels of one pixel, so the
// epilogue stores straight from registers, coalesced.
struct ConvClParams {
    int32_t k_out, c_blocks, kernel_h, kernel_w, pad_y, pad_x;
    int32_t hb, hb_shift, ncols;        // sub-tile rows (power of two), columns = 8 * hb
    int32_t per_cta, tmem_cols, stages;
    int32_t n_mma, col_stride;          // one MMA spans all sub-tiles of the CTA: N columns, columns between sub-tiles
    int32_t tiles_w, tiles_h, subtiles; // sub-tile grid per image and in total
    int32_t n_img, oh, ow;
    int32_t iters;                      // kernel_w * c_blocks
    float* out;
    const float* add1;
    const float* add2;
    int64_t so[4], s1[4], s2[4];        // (n, c, h, w) strides
    int32_t act, round_tf32;
    // bulk-copy epilogue: the residual tile is prefetched into shared memory by the copy engine while
    // the mainloop runs and the finished tile leaves through a bulk tensor store
    int32_t tma_io, has_res;
    int32_t io_alias;                   // the in/out tile reuses a retired pipeline slot instead of its own region
    const float* bias;                  // tma_io: one value per output channel (or null)
    int64_t bias_stride;
    uint32_t* status;
};

constexpr int kMaxPerCta = 8;

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
tc_conv_cl_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                  const __grid_constant__ CUtensorMap map_res, const __grid_constant__ CUtensorMap map_out,
                  const __grid_constant__ ConvClParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int stages = p.stages;
    const uint32_t w_bytes = (uint32_t)p.kernel_h * kATileBytes;                 // R tiles of 128 x 128 B
    const uint32_t x_tile_bytes = (uint32_t)(p.hb + p.kernel_h - 1) * 1024u;     // one sub-tile window
    const uint32_t stage_bytes = w_bytes + (uint32_t)p.per_cta * x_tile_bytes;
    // in/out tile [sub-tile][pixel][128 channels] f32: its own region behind the stages, or (io_alias)
    // the pipeline slot that retires first
    const uint32_t io_tile_bytes = p.tma_io ? (uint32_t)p.ncols * 512u : 0u;
    const uint32_t io_base = p.io_alias ? base + (uint32_t)(p.iters % stages) * stage_bytes : base + (uint32_t)stages * stage_bytes;
    const uint32_t bar_base = base + (uint32_t)stages * stage_bytes + (p.io_alias ? 0u : (uint32_t)p.per_cta * io_tile_bytes);
    const uint32_t full_bar = bar_base, empty_bar = bar_base + 8u * stages, accum_bar = bar_base + 16u * stages;
    const uint32_t res_bar = accum_bar + 8u;
    const uint32_t slot_addr = res_bar + 8u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + (slot_addr - base));
    volatile int* abandon = (volatile int*)(gen_base + (slot_addr + 4u - base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(full_bar + 8u * s, 1);
            mbar_init(empty_bar + 8u * s, 1);
        }
        mbar_init(accum_bar, 1);
        mbar_init(res_bar, 1);
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

    const int k0 = blockIdx.y * kBlockM;             // first output channel of this CTA
    const int first_subtile = blockIdx.x * p.per_cta;

    // Programmatic dependent launch: let the next kernel of the step list be scheduled onto SMs as
    // this grid's CTAs retire (its prologue then overlaps our tail) ...
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0 && lane == 0) {
        // ---------------- producer
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        if (p.tma_io) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_res) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_out) : "memory");
        }
        // ... and, being such a dependent ourselves, touch nothing the previous kernel wrote before it
        // has completed.  Every load is issued by this thread; MMAs and the epilogue follow from them.
        // The filter is a constant of the plan, not an output of the previous kernel: its tiles for the
        // first round of stages are requested before the wait, so their latency overlaps the
        // previous kernel's tail.
        const int early = p.iters < stages ? p.iters : stages;
        for (int it = 0; it < early; it++) {
            const uint32_t bar = full_bar + 8u * it;
            mbar_expect_tx(bar, stage_bytes);
            const int sx = it / p.c_blocks, cb = it - sx * p.c_blocks;
            tma_load_4d(base + (uint32_t)it * stage_bytes, &map_w, bar, cb * kBlockK, k0, sx, 0);
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        auto prefetch_residual = [&]() {
            int valid = p.subtiles - first_subtile;
            if (valid > p.per_cta) valid = p.per_cta;
            mbar_expect_tx(res_bar, (uint32_t)valid * io_tile_bytes);
            for (int i = 0; i < valid; i++) {
                const int sub = first_subtile + i;
                const int tw = sub % p.tiles_w;
                const int th = (sub / p.tiles_w) % p.tiles_h;
                const int img = sub / (p.tiles_w * p.tiles_h);
                tma_load_4d(io_base + (uint32_t)i * io_tile_bytes, &map_res, res_bar, k0, tw * 8, th * p.hb, img);
            }
        };
        if (p.tma_io && p.has_res && !p.io_alias) prefetch_residual();   // own region: as early as possible
        for (int it = 0; it < p.iters; it++) {
            const int st = it % stages;
            const uint32_t parity = ((it / stages) & 1) ^ 1;
            const uint32_t bar = full_bar + 8u * st;
            const int sx = it / p.c_blocks, cb = it - sx * p.c_blocks;
            const uint32_t stage_addr = base + (uint32_t)st * stage_bytes;
            if (it >= early) {
                if (!mbar_wait(empty_bar + 8u * st, parity, abandon, p.status, 1)) break;
                mbar_expect_tx(bar, stage_bytes);
                tma_load_4d(stage_addr, &map_w, bar, cb * kBlockK, k0, sx, 0);
            }
            for (int i = 0; i < p.per_cta; i++) {
                const int sub = first_subtile + i;       // past the end: every coordinate is out of range, zero fill
                const int tw = sub % p.tiles_w;
                const int th = (sub / p.tiles_w) % p.tiles_h;
                const int img = sub / (p.tiles_w * p.tiles_h);
                tma_load_4d(stage_addr + w_bytes + (uint32_t)i * x_tile_bytes, &map_x, bar, cb * kBlockK,
                            tw * 8 + sx - p.pad_x, th * p.hb - p.pad_y, img);
            }
        }
        if (p.tma_io && p.has_res && p.io_alias) {
            // The in/out tile lives in the pipeline slot that retires first: slot iters % stages, which
            // the next iteration would have refilled.  Wait for its last MMA like any refill, then
            // fetch the residual there; it lands while the remaining stages are still being consumed.
            const int it = p.iters, st = it % stages;
            const uint32_t parity = ((it / stages) & 1) ^ 1;
            if (mbar_wait(empty_bar + 8u * st, parity, abandon, p.status, 1)) prefetch_residual();
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer: M = 128 output channels.  The windows of the CTA's sub-tiles lie
        // back to back in the stage, (hb + R - 1) groups of 8 pixels each, so ONE instruction per tap and
        // K step covers all of them: its N spans per_cta * hb + (per_cta - 1) * (R - 1) groups, and the
        // (R - 1) groups between two sub-tiles accumulate values nobody reads.  (An instruction costs
        // about the same for N = 64 as for N = 128, so narrow per-sub-tile instructions would halve
        // the tensor throughput.)
        const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.n_mma >> 3) << 17) | ((uint32_t)(kBlockM >> 4) << 24);
        bool ok = true;
        for (int it = 0; it < p.iters && ok; it++) {
            const int st = it % stages;
            const uint32_t parity = (it / stages) & 1;
            ok = mbar_wait(full_bar + 8u * st, parity, abandon, p.status, 2);
            if (!ok) break;
            tc_fence_after();
            const uint32_t stage_addr = base + (uint32_t)st * stage_bytes;
            for (int r = 0; r < p.kernel_h; r++) {
                const uint64_t dw = smem_desc_sw128(stage_addr + (uint32_t)r * kATileBytes);
                const uint64_t dx = smem_desc_sw128(stage_addr + w_bytes + (uint32_t)r * 1024u);
#pragma unroll
                for (int j = 0; j < kBlockK / 8; j++)
                    mma_tf32(tmem_base, dw + 2u * j, dx + 2u * j, idesc, (it | r | j) != 0 ? 1u : 0u);
            }
            mma_commit(empty_bar + 8u * st);
        }
        if (ok) mma_commit(accum_bar);
    } else if (warp >= 2) {
        // ---------------- epilogue: thread <-> accumulator lane <-> output channel
        const int q = warp & 3;
        const int64_t k = (int64_t)k0 + q * 32 + lane;
        const bool ok = mbar_wait(accum_bar, 0, abandon, p.status, 3);
        tc_fence_after();
        const bool k_valid = k < p.k_out;
        if (p.tma_io) {
            const float bias = (p.bias != nullptr && k_valid) ? p.bias[k * p.bias_stride] : 0.f;
            bool res_ok = ok;
            if (ok && p.has_res) res_ok = mbar_wait(res_bar, 0, abandon, p.status, 4);
            float* io = (float*)(gen_base + (io_base - base));
            // the loop below synchronises the four epilogue warps, so they must agree on entering it:
            // vote (every epilogue thread gets here, its waits being bounded)
            uint32_t all_ok;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t"
                "setp.ne.u32 p, %1, 0;\n\t"
                "bar.red.and.pred q, 2, 128, p;\n\t"
                "selp.u32 %0, 1, 0, q;\n\t}"
                : "=r"(all_ok)
                : "r"((uint32_t)res_ok)
                : "memory");
            if (all_ok) {
                for (int i = 0; i < p.per_cta; i++) {
                    const int sub = first_subtile + i;
                    if (sub >= p.subtiles) break;
                    for (int c0 = 0; c0 < p.ncols; c0 += 32) {
                        uint32_t v[32];
                        tmem_load_32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(i * p.col_stride + c0), v);
                        float* cell = io + ((size_t)(i * p.ncols + c0) * kBlockM) + q * 32 + lane;
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            float val = __uint_as_float(v[j]) + bias;
                            if (p.has_res) val += cell[j * kBlockM];
                            cell[j * kBlockM] = finish(val, p.act, p.round_tf32);
                        }
                    }
                    // this sub-tile is complete: hand it to the copy engine while the next one is computed
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> bulk store
                    asm volatile("bar.sync 1, 128;" ::: "memory");                 // the four epilogue warps
                    if (threadIdx.x == 64) {
                        const int tw = sub % p.tiles_w;
                        const int th = (sub / p.tiles_w) % p.tiles_h;
                        const int img = sub / (p.tiles_w * p.tiles_h);
                        tma_store_4d(&map_out, io_base + (uint32_t)i * io_tile_bytes, k0, tw * 8, th * p.hb, img);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            }
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory must outlive the reads
        } else if (ok) {
            for (int i = 0; i < p.per_cta; i++) {
                const int sub = first_subtile + i;
                if (sub >= p.subtiles) break;
                const int tw = sub % p.tiles_w;
                const int th = (sub / p.tiles_w) % p.tiles_h;
                const int64_t img = sub / (p.tiles_w * p.tiles_h);
                const int64_t base_o = img * p.so[0] + k * p.so[1];
                const int64_t base_1 = img * p.s1[0] + k * p.s1[1];
                const int64_t base_2 = img * p.s2[0] + k * p.s2[1];
                for (int c0 = 0; c0 < p.ncols; c0 += 32) {
                    uint32_t v[32];
                    tmem_load_32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(i * p.col_stride + c0), v);
                    if (!k_valid) continue;
                    float extra[32];
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int oy = th * p.hb + ((c0 + j) >> 3), ox = tw * 8 + ((c0 + j) & 7);
                        const bool valid = oy < p.oh && ox < p.ow;
                        float e = 0.f;
                        if (valid && p.add1) e += p.add1[base_1 + oy * p.s1[2] + ox * p.s1[3]];
                        if (valid && p.add2) e += p.add2[base_2 + oy * p.s2[2] + ox * p.s2[3]];
                        extra[j] = e;
                    }
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int oy = th * p.hb + ((c0 + j) >> 3), ox = tw * 8 + ((c0 + j) & 7);
                        if (oy < p.oh && ox < p.ow)
                            p.out[base_o + oy * p.so[2] + ox * p.so[3]] = finish(__uint_as_float(v[j]) + extra[j], p.act, p.round_tf32);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    KN_CHECK(fn != nullptr, KN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    return fn;
}

// dims / strides innermost first; strides in elements (dims[0] has stride 1)
CUtensorMap make_map(const void* base, int rank, const int64_t* dims, const int64_t* strides, const int* box,
                     bool operand = true, bool atom_32b = false) {
    KN_CHECK(((uintptr_t)base & 15) == 0, KN_ERR_INTERNAL, "TMA base address is not 16-byte aligned");
    cuuint64_t gdim[5], gstride[4];
    cuuint32_t gbox[5], estride[5];
    for (int i = 0; i < rank; i++) {
        gdim[i] = (cuuint64_t)std::max<int64_t>(dims[i], 1);
        gbox[i] = (cuuint32_t)box[i];
        estride[i] = 1;
        if (i > 0) {
            int64_t bytes = strides[i] * 4;
            if (dims[i] <= 1 && (bytes <= 0 || bytes % 16 != 0)) bytes = 16;   // never stepped: any legal value
            KN_CHECK(bytes > 0 && bytes % 16 == 0, KN_ERR_INTERNAL, "TMA stride is not a positive multiple of 16 bytes");
            gstride[i - 1] = (cuuint64_t)bytes;
        }
    }
    CUtensorMap map;
    // TFLOAT32: the copy engine rounds each f32 to TF32 on its way into shared memory, so operands
    // are rounded to nearest instead of being truncated by the tensor core
    // (epilogue tiles, `operand == false`, are plain f32 rows without swizzle)
    CUresult res = encode_tiled_fn()(&map, operand ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                                     (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, gbox, estride,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     operand ? (atom_32b ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B) : CU_TENSOR_MAP_SWIZZLE_NONE,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KN_CHECK(res == CUDA_SUCCESS, KN_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)res));
    return map;
}

int round_up(int x, int to) { return (x + to - 1) / to * to; }
// dynamic shared memory of tc_contract_kernel: operand stages or the staged epilogue's tile (whichever
// is larger), then barriers and control words, plus slack for the 1024-byte alignment of the base
int contract_smem_bytes(int stages, int bn, bool staged) {
    const int operands = stages * (kATileBytes + bn * 128);
    const int staging = staged ? kBlockM * (bn + 4) * 4 : 0;
    return std::max(operands, staging) + 16 * stages + 64 + 1024;
}
int pow2_ceil(int x) {
    int p = 1;
    while (p < x) p <<= 1;
    return p;
}

}  // namespace

struct TcLaunch {
    CUtensorMap map_a, map_b, map_res, map_out;
    TcParams p;
    bool channels_last = false;   // tc_conv_cl_kernel with `cl` instead of tc_contract_kernel with `p`
    bool split_k = false;         // tc_contract_kernel writes partial tiles, splitk_reduce_kernel finishes
    SplitKReduceParams reduce;
    ConvClParams cl;
    dim3 grid;
    int smem_bytes;
    std::shared_ptr<void> chain;  // ConvChain step: launch data of kernels/conv_chain.cu
    std::shared_ptr<void> gemm_p; // matmul taken by the persistent kernel (kernels/gemm_persistent.cu)
    std::shared_ptr<void> attn;   // matmul with a row softmax (kernels/attn_softmax.cu)
    std::shared_ptr<void> attention;   // scores, softmax and probabilities . V (kernels/attention.cu)
};

CUtensorMap tc_make_store_map(const void* base, int rank, const int64_t* dims, const int64_t* strides, const int* box) {
    KN_CHECK(((uintptr_t)base & 15) == 0, KN_ERR_INTERNAL, "TMA base address is not 16-byte aligned");
    cuuint64_t gdim[5], gstride[4];
    cuuint32_t gbox[5], estride[5];
    for (int i = 0; i < rank; i++) {
        gdim[i] = (cuuint64_t)std::max<int64_t>(dims[i], 1);
        gbox[i] = (cuuint32_t)box[i];
        estride[i] = 1;
        if (i > 0) {
            int64_t bytes = strides[i] * 4;
            if (dims[i] <= 1 && (bytes <= 0 || bytes % 16 != 0)) bytes = 16;
            KN_CHECK(bytes > 0 && bytes % 16 == 0, KN_ERR_INTERNAL, "TMA stride is not a positive multiple of 16 bytes");
            gstride[i - 1] = (cuuint64_t)bytes;
        }
    }
    CUtensorMap map;
    CUresult res = encode_tiled_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride,
                                     gbox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KN_CHECK(res == CUDA_SUCCESS, KN_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)res));
    return map;
}

CUtensorMap tc_make_map(const void* base, int rank, const int64_t* dims, const int64_t* strides, const int* box, bool operand) {
    return make_map(base, rank, dims, strides, box, operand);
}
CUtensorMap tc_make_map_mn_major(const void* base, int rank, const int64_t* dims, const int64_t* strides, const int* box) {
    return make_map(base, rank, dims, strides, box, true, true);
}

CUtensorMap tc_make_map_f16(const void* base, int rank, const int64_t* dims, const int64_t* strides, const int* box, bool operand) {
    KN_CHECK(((uintptr_t)base & 15) == 0, KN_ERR_INTERNAL, "TMA base address is not 16-byte aligned");
    cuuint64_t gdim[5], gstride[4];
    cuuint32_t gbox[5], estride[5];
    for (int i = 0; i < rank; i++) {
        gdim[i] = (cuuint64_t)std::max<int64_t>(dims[i], 1);
        gbox[i] = (cuuint32_t)box[i];
        estride[i] = 1;
        if (i > 0) {
            int64_t bytes = strides[i] * 2;
            if (dims[i] <= 1 && (bytes <= 0 || bytes % 16 != 0)) bytes = 16;   // never stepped: any legal value
            KN_CHECK(bytes > 0 && bytes % 16 == 0, KN_ERR_INTERNAL, "TMA stride is not a positive multiple of 16 bytes");
            gstride[i - 1] = (cuuint64_t)bytes;
        }
    }
    CUtensorMap map;
    CUresult res = encode_tiled_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride,
                                     gbox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     operand ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KN_CHECK(res == CUDA_SUCCESS, KN_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)res));
    return map;
}

static bool tma_stride_ok_host(int64_t dim, int64_t stride) { return dim <= 1 || (stride > 0 && stride % 4 == 0); }

// Fills the channels-last convolution launch if the step qualifies: channels-last output, at least
// four output rows, and two pipeline stages of its filter taps fit in shared memory.
static bool prepare_conv_channels_last(const ConvParams& c, uint32_t* status_word, TcLaunch& launch) {
    if (c.s_out[1] != 1 || c.oh < 4) return false;
    ConvClParams& p = launch.cl;
    memset(&p, 0, sizeof(p));
    p.hb = std::min(32, pow2_ceil(c.oh));
    while ((1 << p.hb_shift) < p.hb) p.hb_shift++;
    p.ncols = 8 * p.hb;
    const int w_bytes = c.r * kATileBytes;
    const int x_bytes = (p.hb + c.r - 1) * 1024;
    const int smem_budget = 220 * 1024;
    // bulk-copy epilogue: needs a channels-last output and residual the copy engine can address, and at
    // most one per-channel addend (bias) besides
    auto tile_ok = [&](const float* ptr, const int64_t* st) {
        return ((uintptr_t)ptr & 15) == 0 && st[1] == 1 && tma_stride_ok_host(c.ow, st[3]) && tma_stride_ok_host(c.oh, st[2]) &&
               tma_stride_ok_host(c.n, st[0]);
    };
    auto per_channel = [&](const int64_t* st) { return st[0] == 0 && st[2] == 0 && st[3] == 0; };
    const float* bias = nullptr;
    const float* res = nullptr;
    const int64_t* res_strides = nullptr;
    int64_t bias_stride = 0;
    bool tma_io = tile_ok(c.out, c.s_out);
    const float* adds[2] = {c.add1, c.add2};
    const int64_t* add_strides[2] = {c.s1, c.s2};
    for (int a = 0; a < 2 && tma_io; a++) {
        if (adds[a] == nullptr) continue;
        if (per_channel(add_strides[a]) && bias == nullptr) {
            bias = adds[a];
            bias_stride = add_strides[a][1];
        } else if (tile_ok(adds[a], add_strides[a]) && res == nullptr) {
            res = adds[a];
            res_strides = add_strides[a];
        } else {
            tma_io = false;
        }
    }
    const int io_bytes = tma_io ? p.ncols * 512 : 0;
    if (2 * (w_bytes + x_bytes) + (io_bytes <= w_bytes + x_bytes ? 0 : io_bytes) > smem_budget) return false;
    p.tiles_w = (c.ow + 7) / 8;
    p.tiles_h = (c.oh + p.hb - 1) / p.hb;
    const int64_t subtiles = (int64_t)c.n * p.tiles_w * p.tiles_h;
    if (subtiles > (1ll << 30)) return false;
    p.subtiles = (int)subtiles;
    // sub-tiles per CTA: the filter is fetched once per CTA, the windows once per sub-tile; pick the
    // count that moves the fewest bytes per SM over all waves of a 148-SM device
    const int k_blocks = (c.k + kBlockM - 1) / kBlockM;
    int best = 1;
    double best_cost = 1e300;
    for (int per = 1; per <= kMaxPerCta; per++) {
        const int stage = w_bytes + per * x_bytes;
        const int io_extra = per * io_bytes <= stage ? 0 : per * io_bytes;   // fits a retired slot, or needs its own region
        if (8 * (per * p.hb + (per - 1) * (c.r - 1)) > 256 || 2 * stage + io_extra > smem_budget) break;
        const int64_t ctas = ((subtiles + per - 1) / per) * k_blocks;
        const double waves = (double)((ctas + 147) / 148);
        const double cost = waves * (w_bytes + (double)per * x_bytes);
        if (cost < best_cost) { best_cost = cost; best = per; }
    }
    p.per_cta = best;
    p.col_stride = 8 * (p.hb + c.r - 1);
    p.n_mma = 8 * (p.per_cta * p.hb + (p.per_cta - 1) * (c.r - 1));
    p.tmem_cols = std::max(32, pow2_ceil(p.n_mma));
    const int stage_bytes = w_bytes + p.per_cta * x_bytes;
    // the in/out tile may reuse the first pipeline slot to retire when it fits into one slot
    const bool io_alias = tma_io && p.per_cta * io_bytes <= stage_bytes;
    p.io_alias = io_alias ? 1 : 0;
    p.stages = std::max(2, std::min(4, (smem_budget - (io_alias ? 0 : p.per_cta * io_bytes)) / stage_bytes));
    p.k_out = c.k;
    p.c_blocks = (c.c + kBlockK - 1) / kBlockK;
    p.kernel_h = c.r;
    p.kernel_w = c.s;
    p.pad_y = c.pad_y;
    p.pad_x = c.pad_x;
    p.iters = c.s * p.c_blocks;
    p.stages = std::min(p.stages, std::max(2, p.iters));
    p.n_img = c.n;
    p.oh = c.oh;
    p.ow = c.ow;
    p.out = c.out;
    p.add1 = c.add1;
    p.add2 = c.add2;
    for (int i = 0; i < 4; i++) {
        p.so[i] = c.s_out[i];
        p.s1[i] = c.s1[i];
        p.s2[i] = c.s2[i];
    }
    p.act = c.act;
    p.round_tf32 = c.round_tf32;
    p.status = status_word;
    // filter memory is [tap = r * S + s][out channel][in channel padded to 4]; viewed as (c, k, s, r)
    const int64_t c_pad = round_up(c.c, 4);
    int64_t wdims[4] = {c.c, c.k, c.s, c.r}, wstr[4] = {1, c_pad, c_pad * c.k, c_pad * c.k * c.s};
    int wbox[4] = {kBlockK, kBlockM, 1, c.r};
    launch.map_a = make_map(c.filter, 4, wdims, wstr, wbox);
    int64_t xdims[4] = {c.c, c.w, c.h, c.n}, xstr[4] = {1, c.s_in[3], c.s_in[2], c.s_in[0]};
    int xbox[4] = {kBlockK, 8, p.hb + c.r - 1, 1};
    launch.map_b = make_map(c.in, 4, xdims, xstr, xbox);
    launch.grid = dim3((unsigned)((subtiles + p.per_cta - 1) / p.per_cta), (unsigned)k_blocks, 1);
    p.tma_io = tma_io ? 1 : 0;
    p.has_res = res != nullptr ? 1 : 0;
    p.bias = bias;
    p.bias_stride = bias_stride;
    if (tma_io) {
        int64_t odims[4] = {c.k, c.ow, c.oh, c.n}, ostr[4] = {1, c.s_out[3], c.s_out[2], c.s_out[0]};
        int obox[4] = {kBlockM, 8, p.hb, 1};
        launch.map_out = make_map(c.out, 4, odims, ostr, obox, false);
        launch.map_res = launch.map_out;
        if (res != nullptr) {
            int64_t rstr[4] = {1, res_strides[3], res_strides[2], res_strides[0]};
            launch.map_res = make_map(res, 4, odims, rstr, obox, false);
        }
    } else {
        launch.map_res = launch.map_a;
        launch.map_out = launch.map_a;
    }
    launch.smem_bytes = p.stages * stage_bytes + (p.io_alias ? 0 : p.per_cta * io_bytes) + 16 * p.stages + 64 + 1024;
    launch.channels_last = true;
    return true;
}

bool tc_conv_tile(int oh, int ow, int* wb, int* hb, int* nb) {
    int w = std::min(pow2_ceil(ow), kBlockM);
    int h = std::min(pow2_ceil(oh), kBlockM / w);
    *wb = w;
    *hb = h;
    *nb = kBlockM / (w * h);
    return true;
}

void tc_prepare_step(Step& step, uint32_t* status_word, int flags, uint32_t* trace_words) {
    auto launch = std::make_shared<TcLaunch>();
    if (step.kind == StepKind::ConvChain) {
        launch->chain = chain_prepare(step.chain, status_word);
        step.tc = launch;
        return;
    }
    TcParams& p = launch->p;
    memset(&p, 0, sizeof(p));
    p.status = status_word;
    int64_t n_cols;
    if (step.kind == StepKind::Gemm) {
        const GemmParams& g = step.gemm;
        if (g.row_softmax == 2) {
            launch->attention = attention_prepare(g, status_word);
            KN_CHECK(launch->attention != nullptr, KN_ERR_INTERNAL, "fused attention step does not qualify");
            step.tc = launch;
            return;
        }
        if (g.row_softmax) {
            launch->attn = attn_softmax_prepare(g, status_word);
            KN_CHECK(launch->attn != nullptr, KN_ERR_INTERNAL, "matmul with a row softmax does not qualify");
            step.tc = launch;
            return;
        }
        if (g.half || g.conv_operand != 0 || g.a4.enabled || g.b4.enabled) {
            // f16 storage, or an implicit convolution operand: the persistent kernel is the only tensor-core kernel
            // that takes these; the planner marks such a step tensor-core only when that kernel takes it
            int per_slice = 0, splits = 1;
            if (g.splits > 1) {
                const int block_k = g.half ? 64 : 32;
                const int k_total = (int)((g.k + block_k - 1) / block_k);
                per_slice = (k_total + g.splits - 1) / g.splits;
                splits = (k_total + per_slice - 1) / per_slice;
            }
            launch->gemm_p = gemm_persistent_prepare(g, status_word, splits, per_slice, trace_words);
            KN_CHECK(launch->gemm_p != nullptr, KN_ERR_INTERNAL,
                     g.half ? "f16 matmul planned for the tensor cores does not qualify"
                            : "matmul with an operand read in place (convolution windows, head split or merge) does not qualify");
            if (splits > 1) {
                SplitKReduceParams& r = launch->reduce;
                memset(&r, 0, sizeof(r));
                r.partial = g.scratch;
                r.splits = splits;
                r.batch = g.batch;
                r.m = g.m;
                r.n = g.n;
                r.out = g.c;
                r.add1 = g.add1;
                r.add2 = g.add2;
                for (int i = 0; i < 3; i++) {
                    r.so[i] = g.sc[i];
                    r.s1[i] = g.s1[i];
                    r.s2[i] = g.s2[i];
                }
                r.act = g.act;
                r.half = g.half;
                r.round_tf32 = g.round_tf32;
                launch->split_k = true;
            }
            step.tc = launch;
            return;
        }
        if (g.splits <= 1 && !(flags & KN_FLAG_NO_PERSISTENT_GEMM)) {
            launch->gemm_p = gemm_persistent_prepare(g, status_word, 1, 0, trace_words);
            if (launch->gemm_p) {
                step.tc = launch;
                return;
            }
        }
        p.mode = 0;
        n_cols = g.n;
        p.m = g.m;
        p.n = g.n;
        p.k_iters = (int)((g.k + kBlockK - 1) / kBlockK);
        p.out = g.c;
        p.add1 = g.add1;
        p.add2 = g.add2;
        for (int i = 0; i < 3; i++) {
            p.so[i] = g.sc[i];
            p.s1[i] = g.s1[i];
            p.s2[i] = g.s2[i];
        }
        p.act = g.act;
        p.round_tf32 = g.round_tf32;
        // A: [batch, m, k] with k contiguous; B: [batch, k, n] with k contiguous
        p.a_batch = (g.batch > 1 && g.sa[0] == 0) ? 0 : 1;
        int64_t adims[4] = {g.k, g.m, p.a_batch ? g.batch : 1, 1}, astr[4] = {1, g.sa[1], p.a_batch ? g.sa[0] : 4, 4};
        int abox[4] = {kBlockK, kBlockM, 1, 1};
        launch->map_a = make_map(g.a, 4, adims, astr, abox);
        p.bn = (int)std::min<int64_t>(round_up((int)std::min<int64_t>(n_cols, 256), 16), 256);
        if (n_cols > 256) p.bn = 128;
        p.b_batch = (g.batch > 1 && g.sb[0] == 0) ? 0 : 1;
        int64_t bdims[3] = {g.k, g.n, p.b_batch ? g.batch : 1}, bstr[3] = {1, g.sb[2], p.b_batch ? g.sb[0] : 4};
        int bbox[3] = {kBlockK, p.bn, 1};
        launch->map_b = make_map(g.b, 3, bdims, bstr, bbox);
        launch->grid = dim3((unsigned)((g.m + kBlockM - 1) / kBlockM), (unsigned)((n_cols + p.bn - 1) / p.bn), (unsigned)g.batch);
        p.k_iters_total = p.k_iters;
        p.splits = 1;
        if (g.splits > 1) {
            // split K: every slice writes a dense [m][n] partial tile into the step's scratch buffer,
            // splitk_reduce_kernel sums the slices and applies the epilogue
            const int per_slice = (p.k_iters_total + g.splits - 1) / g.splits;
            p.k_iters = per_slice;
            p.splits = (p.k_iters_total + per_slice - 1) / per_slice;   // no empty slice
            SplitKReduceParams& r = launch->reduce;
            memset(&r, 0, sizeof(r));
            r.partial = g.scratch;
            r.splits = p.splits;
            r.batch = g.batch;
            r.m = g.m;
            r.n = g.n;
            r.out = g.c;
            r.add1 = g.add1;
            r.add2 = g.add2;
            for (int i = 0; i < 3; i++) {
                r.so[i] = g.sc[i];
                r.s1[i] = g.s1[i];
                r.s2[i] = g.s2[i];
            }
            r.act = g.act;
            r.round_tf32 = g.round_tf32;
            p.out = g.scratch;
            p.add1 = nullptr;
            p.add2 = nullptr;
            p.act = 0;
            p.round_tf32 = 0;
            p.so[0] = g.m * g.n;   // per (batch, slice)
            p.so[1] = g.n;
            p.so[2] = 1;
            launch->grid.z = (unsigned)(g.batch * p.splits);
            launch->split_k = true;
            // the partial tiles can come from the persistent kernel too (its epilogue hands whole 128 x 32
            // blocks to the copy engine instead of storing row by row)
            if (!(flags & KN_FLAG_NO_PERSISTENT_GEMM)) launch->gemm_p = gemm_persistent_prepare(g, status_word, p.splits, per_slice, trace_words);
        }
    } else {
        const ConvParams& c = step.conv;
        if (prepare_conv_channels_last(c, status_word, *launch)) {
            step.tc = launch;
            return;
        }
        p.mode = 1;
        n_cols = c.k;
        p.n = c.k;
        p.cblocks = (c.c + kBlockK - 1) / kBlockK;
        p.k_iters = c.r * c.s * p.cblocks;
        p.k_iters_total = p.k_iters;
        p.splits = 1;
        p.kernel_w = c.s;
        p.pad_y = c.pad_y;
        p.pad_x = c.pad_x;
        tc_conv_tile(c.oh, c.ow, &p.wb, &p.hb, &p.nb);
        while ((1 << p.wb_shift) < p.wb) p.wb_shift++;
        while ((1 << p.hb_shift) < p.hb) p.hb_shift++;
        p.tiles_w = (c.ow + p.wb - 1) / p.wb;
        p.tiles_h = (c.oh + p.hb - 1) / p.hb;
        const int tiles_n = (c.n + p.nb - 1) / p.nb;
        p.n_img = c.n;
        p.oh = c.oh;
        p.ow = c.ow;
        p.out = c.out;
        p.add1 = c.add1;
        p.add2 = c.add2;
        for (int i = 0; i < 4; i++) {
            p.so[i] = c.s_out[i];
            p.s1[i] = c.s1[i];
            p.s2[i] = c.s2[i];
        }
        p.act = c.act;
        p.round_tf32 = c.round_tf32;
        // input viewed as (C, W, H, N), channels contiguous
        int64_t adims[4] = {c.c, c.w, c.h, c.n}, astr[4] = {1, c.s_in[3], c.s_in[2], c.s_in[0]};
        int abox[4] = {kBlockK, p.wb, p.hb, p.nb};
        launch->map_a = make_map(c.in, 4, adims, astr, abox);
        p.bn = (int)std::min<int64_t>(round_up((int)std::min<int64_t>(n_cols, 256), 16), 256);
        if (n_cols > 256) p.bn = 128;
        // filter stored as (tap, out channel, in channel) with in-channel rows padded to a multiple of 4
        const int64_t c_pad = round_up(c.c, 4);
        int64_t bdims[3] = {c.c, c.k, (int64_t)c.r * c.s}, bstr[3] = {1, c_pad, c_pad * c.k};
        int bbox[3] = {kBlockK, p.bn, 1};
        launch->map_b = make_map(c.filter, 3, bdims, bstr, bbox);
        launch->grid = dim3((unsigned)(p.tiles_w * p.tiles_h * tiles_n), (unsigned)((n_cols + p.bn - 1) / p.bn), 1);
    }
    p.tmem_cols = std::max(32, pow2_ceil(p.bn));
    const int stage_bytes = kATileBytes + p.bn * 128;
    p.stages = std::max(2, std::min(6, (200 * 1024) / stage_bytes));
    p.stages = std::min(p.stages, std::max(2, p.k_iters));
    p.staged = (p.mode == 0 ? p.so[2] : p.so[1]) == 1 ? 1 : 0;
    {
        // rows are (batch, row) for matmul and (image, y, x) for conv; columns are the remaining stride
        auto classify = [&](const float* ptr, const int64_t* st) -> int {
            if (ptr == nullptr) return 0;
            const int64_t col = p.mode == 0 ? st[2] : st[1];
            const int64_t r0 = st[0], r1 = p.mode == 0 ? st[1] : st[2], r2 = p.mode == 0 ? 0 : st[3];
            if (col != 1 || ((uintptr_t)ptr & 15) != 0) return 3;
            if (r0 == 0 && r1 == 0 && r2 == 0) return 1;
            if (r0 % 4 == 0 && r1 % 4 == 0 && r2 % 4 == 0) return 2;
            return 3;
        };
        p.add1_mode = classify(p.add1, p.s1);
        p.add2_mode = classify(p.add2, p.s2);
        const int out_mode = classify(p.out, p.so);
        p.vec4 = p.staged && p.n % 4 == 0 && out_mode == 2 && p.add1_mode != 3 && p.add2_mode != 3;
    }
    launch->smem_bytes = contract_smem_bytes(p.stages, p.bn, p.staged != 0);
    step.tc = launch;
}

static int launch_splitk_reduce(const SplitKReduceParams& r, cudaStream_t stream) {
    const int64_t total = r.batch * r.m * r.n;
    const unsigned blocks = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8);
    launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), (size_t)(0), stream, r);
    return (int)cudaGetLastError();
}

int tc_launch_step(const Step& step, cudaStream_t stream) {
    const TcLaunch& l = *step.tc;
    if (l.chain) return chain_launch(l.chain.get(), stream);
    if (l.attention) return attention_launch(l.attention.get(), stream);
    if (l.attn) return attn_softmax_launch(l.attn.get(), stream);
    if (l.gemm_p) {
        const int err = gemm_persistent_launch(l.gemm_p.get(), stream);
        if (err != 0 || !l.split_k) return err;
        return launch_splitk_reduce(l.reduce, stream);
    }
    // the opt-in to large dynamic shared memory is per device
    static std::mutex mu;
    static bool done[64] = {false};
    int device = 0;
    cudaGetDevice(&device);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (device >= 0 && device < 64 && !done[device]) {
            cudaError_t e1 = cudaFuncSetAttribute(tc_contract_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            cudaError_t e2 = cudaFuncSetAttribute(tc_conv_cl_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e1 != cudaSuccess) return (int)e1;
            if (e2 != cudaSuccess) return (int)e2;
            done[device] = true;
        }
    }
    if (l.grid.x == 0 || l.grid.y == 0 || l.grid.z == 0) return 0;
    if (l.channels_last) {
        // may start while the previous kernel of the stream drains (see griddepcontrol in the kernel)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = l.grid;
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = (size_t)l.smem_bytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        return (int)cudaLaunchKernelEx(&cfg, tc_conv_cl_kernel, l.map_a, l.map_b, l.map_res, l.map_out, l.cl);
    }
    launch_pdl(tc_contract_kernel, dim3(l.grid), dim3(kThreads), (size_t)(l.smem_bytes), stream, l.map_a, l.map_b, l.p);
    if (l.split_k) return launch_splitk_reduce(l.reduce, stream);
    return (int)cudaGetLastError();
}

}  // namespace kn

// ------------------------------------------------------------------------------------------------
// Matrix multiply for callers that must not allocate
// ------------------------------------------------------------------------------------------------
// Some hosts of this library run where device allocation is off the table: inside a latency-critical
// serving loop that has promised its allocator a fixed footprint, from a plugin callback of a runtime
// that owns all device memory, or on a context whose memory pool is already carved up.  The executor's
// split-K matmul keeps its partial tiles in the arena it allocated; this entry point runs the same two
// kernels with the partial tiles in a fixed array that is part of the loaded module instead, so a call
// allocates nothing (no cudaMalloc / cudaFree, no allocating library routine).  The price: the array
// occupies KN_STATIC_SCRATCH_BYTES on every GPU that loads the library until the process exits, and it
// caps the problem size.
namespace kn {
namespace {

constexpr size_t kStaticScratchFloats = (size_t)KN_STATIC_SCRATCH_BYTES / 4;

// Device-resident scratch.  In host code these names are host-side stand-ins, NOT device addresses:
// the device addresses are fetched once per device with cudaGetSymbolAddress (below).
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
static __device__ __align__(256) uint32_t g_static_status[64];

struct StaticDevice {
    bool ready = false;
    float* scratch = nullptr;
    uint32_t* status = nullptr;
};
std::mutex g_static_mu;
StaticDevice g_static_dev[64];

// One-time set-up for the current device: resolve the device addresses of the two arrays and opt the
// kernel in to large dynamic shared memory.  None of this allocates device memory.
const StaticDevice& static_device_setup() {
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    KN_CHECK(err == cudaSuccess, KN_ERR_CUDA, std::string("cudaGetDevice failed: ") + cudaGetErrorString(err));
    KN_CHECK(device >= 0 && device < 64, KN_ERR_UNSUPPORTED, "device index above 63");
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticDevice& d = g_static_dev[device];
    if (!d.ready) {
        void* scratch = nullptr;
        void* status = nullptr;
        err = cudaGetSymbolAddress(&scratch, g_static_scratch);
        KN_CHECK(err == cudaSuccess && scratch != nullptr, KN_ERR_CUDA,
                 std::string("cudaGetSymbolAddress(scratch) failed: ") + cudaGetErrorString(err));
        err = cudaGetSymbolAddress(&status, g_static_status);
        KN_CHECK(err == cudaSuccess && status != nullptr, KN_ERR_CUDA,
                 std::string("cudaGetSymbolAddress(status) failed: ") + cudaGetErrorString(err));
        err = cudaFuncSetAttribute(tc_contract_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        KN_CHECK(err == cudaSuccess, KN_ERR_CUDA, std::string("cudaFuncSetAttribute failed: ") + cudaGetErrorString(err));
        d.scratch = (float*)scratch;
        d.status = (uint32_t*)status;
        d.ready = true;
    }
    return d;
}

void matmul_static(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k, cudaStream_t stream) {
    KN_CHECK(a != nullptr && b != nullptr && c != nullptr, KN_ERR_INVALID_ARG, "null operand");
    KN_CHECK(m >= 1 && n >= 1 && k >= 1 && m <= (1ll << 30) && n <= (1ll << 30) && k <= (1ll << 30), KN_ERR_INVALID_ARG,
             "matrix extent out of range");
    KN_CHECK(k % 4 == 0, KN_ERR_UNSUPPORTED, "k must be a multiple of 4 (rows of A and B must be 16-byte aligned)");
    KN_CHECK(((uintptr_t)a & 15) == 0 && ((uintptr_t)b & 15) == 0 && ((uintptr_t)c & 3) == 0, KN_ERR_INVALID_ARG,
             "A and B must be 16-byte aligned, C 4-byte aligned");

    // The slicing rule of this entry point (stated in kn_b200.h; the executor's planner uses a rule of its own):
    // column tiles of bn = 128 when n > 256, else n rounded up to 16; K in 32-element blocks; enough slices to
    // reach about 96 CTAs, at least 4 K blocks per slice, at most 32 slices, no empty slice.
    const int bn = n > 256 ? 128 : (int)std::min<int64_t>(round_up((int)std::min<int64_t>(n, 256), 16), 256);
    const int64_t tiles = ((m + kBlockM - 1) / kBlockM) * ((n + bn - 1) / bn);
    const int64_t k_blocks = (k + kBlockK - 1) / kBlockK;
    int64_t splits = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(k_blocks / 4, (96 + tiles - 1) / tiles), 32));
    const int64_t per_slice = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + per_slice - 1) / per_slice;
    const size_t need = (size_t)splits * (size_t)m * (size_t)n;
    KN_CHECK(need <= kStaticScratchFloats, KN_ERR_UNSUPPORTED,
             "problem too large for the static scratch: " + std::to_string(splits) + " K slices x " + std::to_string(m) + " x " +
                 std::to_string(n) + " partial sums need " + std::to_string(need * 4) + " bytes, the limit is " +
                 std::to_string((size_t)KN_STATIC_SCRATCH_BYTES));
    KN_CHECK((m + kBlockM - 1) / kBlockM <= 0x7FFFFFFFll && (n + bn - 1) / bn <= 65535, KN_ERR_UNSUPPORTED, "grid too large");

    const StaticDevice& dev = static_device_setup();

    TcParams p;
    memset(&p, 0, sizeof(p));
    p.mode = 0;
    p.m = m;
    p.n = n;
    p.bn = bn;
    p.tmem_cols = std::max(32, pow2_ceil(bn));
    p.k_iters_total = (int)k_blocks;
    p.k_iters = (int)per_slice;
    p.splits = (int)splits;
    p.out = dev.scratch;            // every (slice, row, column) below m x n is overwritten: nothing to clear
    p.so[0] = m * n;
    p.so[1] = n;
    p.so[2] = 1;
    p.status = dev.status;
    p.a_batch = 1;
    p.b_batch = 1;
    const int stage_bytes = kATileBytes + bn * 128;
    p.stages = std::max(2, std::min(6, (200 * 1024) / stage_bytes));
    p.stages = std::min(p.stages, std::max(2, p.k_iters));
    {
        auto classify_out = [&]() { return ((uintptr_t)p.out & 15) == 0 && n % 4 == 0; };
        p.staged = 1;
        p.vec4 = classify_out() ? 1 : 0;
        p.add1_mode = 0;
        p.add2_mode = 0;
    }
    const int smem_bytes = contract_smem_bytes(p.stages, bn, true);

    int64_t adims[4] = {k, m, 1, 1}, astr[4] = {1, k, 4, 4};
    int abox[4] = {kBlockK, kBlockM, 1, 1};
    const CUtensorMap map_a = make_map(a, 4, adims, astr, abox);
    int64_t bdims[3] = {k, n, 1}, bstr[3] = {1, k, 4};
    int bbox[3] = {kBlockK, bn, 1};
    const CUtensorMap map_b = make_map(b, 3, bdims, bstr, bbox);

    SplitKReduceParams r;
    memset(&r, 0, sizeof(r));
    r.partial = dev.scratch;
    r.splits = (int)splits;
    r.batch = 1;
    r.m = m;
    r.n = n;
    r.out = c;
    r.so[0] = m * n;
    r.so[1] = n;
    r.so[2] = 1;

    dim3 grid((unsigned)((m + kBlockM - 1) / kBlockM), (unsigned)((n + bn - 1) / bn), (unsigned)splits);
    launch_pdl(tc_contract_kernel, dim3(grid), dim3(kThreads), (size_t)(smem_bytes), stream, map_a, map_b, p);
    cudaError_t err = cudaGetLastError();
    KN_CHECK(err == cudaSuccess, KN_ERR_CUDA, std::string("launch failed: ") + cudaGetErrorString(err));
    const int64_t total = m * n;
    const unsigned blocks = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8);
    launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), (size_t)(0), stream, r);
    err = cudaGetLastError();
    KN_CHECK(err == cudaSuccess, KN_ERR_CUDA, std::string("launch failed: ") + cudaGetErrorString(err));
}

// Reads the status word of the current device and clears it.  The word is raised by a kernel of
// kn_matmul_tf32_static whose bounded barrier wait ran out (that CTA then skipped its part of the result).
// Two 4-byte copies between the module's array and the host: nothing is allocated.
int matmul_static_status() {
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    KN_CHECK(err == cudaSuccess, KN_ERR_CUDA, std::string("cudaGetDevice failed: ") + cudaGetErrorString(err));
    KN_CHECK(device >= 0 && device < 64, KN_ERR_UNSUPPORTED, "device index above 63");
    uint32_t* word = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mu);
        if (!g_static_dev[device].ready) return 0;   // no call has run on this device yet
        word = g_static_dev[device].status;
    }
    uint32_t code = 0;
    err = cudaMemcpy(&code, word, sizeof(code), cudaMemcpyDeviceToHost);
    KN_CHECK(err == cudaSuccess, KN_ERR_CUDA, std::string("reading the status word failed: ") + cudaGetErrorString(err));
    if (code != 0) {
        const uint32_t zero = 0;
        err = cudaMemcpy(word, &zero, sizeof(zero), cudaMemcpyHostToDevice);
        KN_CHECK(err == cudaSuccess, KN_ERR_CUDA, std::string("clearing the status word failed: ") + cudaGetErrorString(err));
    }
    return (int)code;
}

}  // namespace
}  // namespace kn

extern "C" KN_API int kn_matmul_tf32_static_status(int* code) {
    try {
        KN_CHECK(code != nullptr, KN_ERR_INVALID_ARG, "null code pointer");
        *code = kn::matmul_static_status();
        return KN_OK;
    } catch (const kn::Error& e) {
        kn::set_last_error(e.what());
        return e.code;
    } catch (const std::exception& e) {
        kn::set_last_error(e.what());
        return KN_ERR_INTERNAL;
    }
}

extern "C" KN_API int kn_matmul_tf32_static(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                                            void* stream) {
    try {
        kn::matmul_static(a, b, c, m, n, k, (cudaStream_t)stream);
        return KN_OK;
    } catch (const kn::Error& e) {
        kn::set_last_error(e.what());
        return e.code;
    } catch (const std::exception& e) {
        kn::set_last_error(e.what());
        return KN_ERR_INTERNAL;
    }
}
