// Consumer loop for units of up to 16 query rows (decode, small GQA groups): every consumer warp owns 16
// tokens of each 128-token tile from score to output accumulation, with its own running max / sum and its
// own O^T[D x rows] accumulators, so consumer warps never meet at a barrier inside the tile loop and drift
// apart to hide each other's latencies.  The eight partial states are combined once per (unit, head) part.
// Part descriptors and Q rows arrive in shared memory from the producer warp, so a part starts without a
// round trip to global memory.  Included by attn_tiled.cu after Cfg, TiledParams, PartDesc and the helpers.
#pragma once

namespace emlx {

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
// the final merge of a unit shared by the consumer warps (see MergeJob)
constexpr int kHelpParts = 128;  // longest list of parts the job area holds
constexpr int kHelpMinParts = 6; // below this the one-warp fold is as fast
constexpr int kMiscHelpExit = 8; // misc[]: the merge warp has left, parked warps may go
template <int D, int NT, int FMT, bool BF16, bool PEER>
__device__ __forceinline__ void park_consumer_warp(const TiledParams& p, uint8_t* fixed, uint64_t* full,
                                                   volatile int* abort_word);
template <bool BF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    uint32_t r;
    if constexpr (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// 2^x on the special-function unit; ex2(-inf) = 0
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float2 h2_to_f2(uint32_t v) {
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

template <int D, int NT, int FMT, bool BF16, bool PEER, bool HELP>
__device__ __forceinline__ void consumer_loop_private(const TiledParams& p, uint8_t* stages, uint8_t* fixed,
                                                      uint64_t* full, uint64_t* empty, volatile int* abort_word,
                                                      long long f_begin, long long f_end, long long total_flat,
                                                      long long active) {
    using C = Cfg<D, NT, FMT>;
    constexpr int KS = D / 16, MT = D / 16, ROWS = C::ROWS, GROUPS = C::GROUPS;
    constexpr int NG = FMT == 0 ? 1 : GROUPS;
    constexpr int RC = C::RED_COLS, RSTRIDE = RC + 4;  // columns of D per cross-warp pass, padded row of the buffer
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    float* ored = (float*)(fixed + C::PBYTES);        // [warps][ROWS][RC + 4]
    float* wm = (float*)(fixed + C::OFF_W);           // [warps][32] per-warp running max
    float* wl = wm + kConsumerWarps * 32;             // [warps][32] per-warp running sum
    float* wb = wl + kConsumerWarps * 32;             // [2][warps][32] per-warp bias terms of the values
    int* misc = (int*)(fixed + C::OFF_MISC);
    bool peer_seen = false;
    uint64_t* dfull = full + 16;
    uint64_t* dempty = full + 20;

    // token of the tile that MMA row g (and g + 8) of this warp stands for; the affine formats permute
    // tokens so that the transposed probabilities line up with the way value codes are unpacked
    const int tokA = 16 * warp + (FMT == 0 ? g : (FMT == 8 ? 4 * (g >> 1) + (g & 1) : 4 * (g >> 1) + 2 * (g & 1)));
    const int tokB = tokA + (FMT == 0 ? 8 : (FMT == 8 ? 2 : 1));

    // ---- per-thread shared-memory offsets inside a stage (they do not change from tile to tile)
    uint32_t k_off = 0, v_off = 0, kq_off[2][NG > 0 ? NG : 1];
    if constexpr (FMT == 0) {
        // ldmatrix rows of K: token 16w + lane%16, 16-byte chunk (k-step, lane/16); XOR swizzle on bits 4..6
        k_off = (uint32_t)((16 * warp + (lane & 15)) * 128 + ((((lane >> 4) ^ (lane & 7)) & 7) << 4));
        // ldmatrix.trans rows of V: token 16w + lane%8 + 8*(lane/16), chunk (2*mt + (lane/8)%2)
        v_off = (uint32_t)(C::KBYTES + (16 * warp + (lane & 7) + 8 * (lane >> 4)) * 128 +
                           (((((lane >> 3) & 1) ^ (lane & 7)) & 7) << 4));
    } else {
        constexpr int KCH = FMT == 8 ? 16 : 8;  // bytes of K codes a thread reads per group and token
#pragma unroll
        for (int j = 0; j < NG; ++j) {
            const int byte = (FMT == 8 ? 64 : 32) * j + KCH * t;
            kq_off[0][j] = ptx::swz<C::KSW>((uint32_t)(tokA * C::KROW + byte));
            kq_off[1][j] = ptx::swz<C::KSW>((uint32_t)(tokB * C::KROW + byte));
        }
        // V^T rows d = 16*mt + g (+8): the swizzle term does not depend on mt
        const int vbyte = FMT == 8 ? 16 * warp + 4 * t : 8 * warp + 2 * t;
        v_off = C::KBYTES + ptx::swz<C::VSW>((uint32_t)(g * C::VROW + vbyte));
    }
    (void)k_off; (void)kq_off;

    uint64_t* mfull = full + 24;
    long long remaining = f_end - f_begin;  // the producer decides the order of the parts; only their total is fixed
    uint32_t it = 0, part_idx = 0;
    int posted = 0;
    bool may_help = false;  // uniform over the CTA's consumer warps

    while (remaining > 0) {
        // ------------------------------------------------------------------ part descriptor from the producer
#ifdef EMLX_TRACE_PARTS
        long long trace_a = 0, trace_b = 0, trace_c = 0, trace_d = 0;
        if (p.trace && tid == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(trace_a));
#endif
        const uint32_t dslot = part_idx % C::NDESC;
        ptx::mbar_wait(&dfull[dslot], (part_idx / C::NDESC) & 1, abort_word);
#ifdef EMLX_TRACE_PARTS
        if (p.trace && tid == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(trace_b));
#endif
        const PartDesc* desc = (const PartDesc*)(fixed + (size_t)dslot * C::DESC_BYTES);
        const int row0 = desc->row0, tile_lo = desc->tile_lo, qs = desc->qs, q_len = desc->q_len;
        const int kv_len = desc->kv_len, head = desc->head, unit = desc->u, j_first = desc->j, run = desc->run;
        const int ntiles = desc->ntiles, cum_u = desc->cum_u;
        const int R = q_len * p.G, ctx = kv_len - q_len;
        const int rows_here = min(ROWS, R - row0);

        int row_hi[NT][2], row_lo[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int rr = min(row0 + 8 * nt + 2 * t + e, R - 1);
                const int i = rr / p.G;
                int hi = min(kv_len, ctx + i + 1);
                int lo = p.window > 0 ? max(0, min(kv_len - 1, ctx + i) - p.window + 1) : 0;
                if (hi <= 0) { hi = 0; lo = 0; }
                row_hi[nt][e] = hi;
                row_lo[nt][e] = lo;
            }
        const int i_first = row0 / p.G, i_last = (row0 + rows_here - 1) / p.G;
        const int hi_min = min(kv_len, ctx + i_first + 1);
        const int lo_max = p.window > 0 ? max(0, min(kv_len - 1, ctx + i_last) - p.window + 1) : 0;

        // Q^T fragments (B operand) from the staged rows; rows past the unit's last one are zero
        uint32_t qf[KS][NT][2];
        float qsum[NG][NT][2];
        {
            const uint8_t* qtile = (const uint8_t*)desc + 64;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const bool ok = 8 * nt + g < rows_here;
                const uint16_t* qrow = (const uint16_t*)(qtile + (size_t)(8 * nt + g) * C::QSTRIDE);
                if constexpr (FMT == 0) {
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks) {
                        qf[ks][nt][0] = ok ? *(const uint32_t*)(qrow + 16 * ks + 2 * t) : 0u;
                        qf[ks][nt][1] = ok ? *(const uint32_t*)(qrow + 16 * ks + 2 * t + 8) : 0u;
                    }
                } else if constexpr (FMT == 8) {
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks) {
                        const uint2 v = ok ? *(const uint2*)(qrow + 64 * (ks >> 2) + 16 * t + 4 * (ks & 3)) : make_uint2(0u, 0u);
                        qf[ks][nt][0] = v.x;
                        qf[ks][nt][1] = v.y;
                    }
                } else {
                    // eight queries q0..q7 face the eight nibbles of one word of key codes, which are unpacked as
                    // (e0,e4) (e1,e5)*16 | (e2,e6) (e3,e7)*16: see unpack_nibbles
#pragma unroll
                    for (int jx = 0; jx < KS / 2; ++jx) {
                        const uint4 v = ok ? *(const uint4*)(qrow + 64 * (jx >> 1) + 16 * t + 8 * (jx & 1)) : make_uint4(0u, 0u, 0u, 0u);
                        qf[2 * jx][nt][0] = ptx::prmt(v.x, v.z, 0x5410u);      // (q0, q4)
                        qf[2 * jx][nt][1] = ptx::prmt(v.x, v.z, 0x7632u);      // (q1, q5)
                        qf[2 * jx + 1][nt][0] = ptx::prmt(v.y, v.w, 0x5410u);  // (q2, q6)
                        qf[2 * jx + 1][nt][1] = ptx::prmt(v.y, v.w, 0x7632u);  // (q3, q7)
                    }
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&dempty[dslot]);
        }
        if constexpr (FMT != 0 && BF16) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    qf[ks][nt][0] = bf16x2_to_f16x2(qf[ks][nt][0]);
                    qf[ks][nt][1] = bf16x2_to_f16x2(qf[ks][nt][1]);
                }
        }
        if constexpr (FMT == 4) {
            // the codes in the upper nibble of a byte arrive 16 times too large: their queries are scaled down instead
            const __half2 sixteenth = __float2half2_rn(0.0625f);
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&qf[ks][nt][1]), sixteenth);
                    qf[ks][nt][1] = *reinterpret_cast<const uint32_t*>(&v);
                }
        }
        if constexpr (FMT != 0) {
            // column sums of Q per scale group through a constant A operand (16 where the queries were scaled down)
            constexpr uint32_t kOne = 0x3C003C00u, kUp = FMT == 4 ? 0x4C004C00u : 0x3C003C00u;
            const uint32_t ones[4] = {kOne, kOne, kUp, kUp};
#pragma unroll
            for (int j = 0; j < NG; ++j)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int sidx = 0; sidx < 4; ++sidx) ptx::mma_16816<false>(c, ones, qf[4 * j + sidx][nt]);
                    qsum[j][nt][0] = c[0];
                    qsum[j][nt][1] = c[1];
                }
        }

        float m[NT][2], l[NT][2], o[MT][NT][4], bsum[NG][NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            m[nt][0] = m[nt][1] = -INFINITY;
            l[nt][0] = l[nt][1] = 0.f;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) o[mt][nt][0] = o[mt][nt][1] = o[mt][nt][2] = o[mt][nt][3] = 0.f;
#pragma unroll
            for (int j = 0; j < NG; ++j) bsum[j][nt][0] = bsum[j][nt][1] = 0.f;
        }

#ifdef EMLX_TRACE_PARTS
        if (p.trace && tid == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(trace_c));
#endif
        for (int jj = 0; jj < run; ++jj, ++it) {
            const uint32_t stage = it % C::STAGES;
            uint8_t* st = stages + (size_t)stage * C::STAGE;
            const uint32_t st_base = ptx::smem_u32(st);
            const __half* sbs = (const __half*)(st + C::KBYTES + C::VBYTES);
            const int t0 = (tile_lo + j_first + jj) * kTile;
            const bool interior = (t0 + kTile <= hi_min) && (t0 >= lo_max);
            ptx::mbar_wait(&full[stage], (it / C::STAGES) & 1, abort_word);
#ifdef EMLX_TRACE_PARTS
            if (p.trace && tid == 0 && jj == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(trace_d));
#endif
#ifdef EMLX_TRACE_TIMELINE
            if (p.trace && tid == 0 && it == 0) {
                long long now;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                p.trace[2048 + 4 * blockIdx.x + 1] = now;
            }
#endif
#ifdef EMLX_EXPERIMENT_STREAM_ONLY  // measurement aid: consume the tiles without any arithmetic
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty[stage]);
            continue;
#endif

            // ---- scores of this warp's 16 tokens against every row
            float s[NT][4];
            if constexpr (FMT == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    uint32_t a[4];
                    ptx::ldmatrix_x4(a, st_base + (ks >> 2) * (kTile * 128) + (k_off ^ (uint32_t)(((ks & 3) * 2) << 4)));
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) ptx::mma_16816<BF16>(s[nt], a, qf[ks][nt]);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) s[nt][c] *= p.scale_log2e;
            } else {
                float acc[NG][NT][4];
#pragma unroll
                for (int j = 0; j < NG; ++j) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) acc[j][nt][0] = acc[j][nt][1] = acc[j][nt][2] = acc[j][nt][3] = 0.f;
                    if constexpr (FMT == 8) {
                        const uint4 xa = *(const uint4*)(st + kq_off[0][j]);
                        const uint4 xb = *(const uint4*)(st + kq_off[1][j]);
                        const uint32_t wa[4] = {xa.x, xa.y, xa.z, xa.w}, wbv[4] = {xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                        for (int sidx = 0; sidx < 4; ++sidx) {
                            const uint32_t a[4] = {ptx::prmt(wa[sidx], 0u, 0x4140u), ptx::prmt(wbv[sidx], 0u, 0x4140u),
                                                   ptx::prmt(wa[sidx], 0u, 0x4342u), ptx::prmt(wbv[sidx], 0u, 0x4342u)};
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) ptx::mma_16816<false>(acc[j][nt], a, qf[4 * j + sidx][nt]);
                        }
                    } else {
                        const uint2 xa = *(const uint2*)(st + kq_off[0][j]);
                        const uint2 xb = *(const uint2*)(st + kq_off[1][j]);
                        const uint32_t wa[2] = {xa.x, xa.y}, wbv[2] = {xb.x, xb.y};
#pragma unroll
                        for (int x = 0; x < 2; ++x) {
                            uint32_t ha[4], hb[4];
                            unpack_nibbles(wa[x], ha);
                            unpack_nibbles(wbv[x], hb);
#pragma unroll
                            for (int y = 0; y < 2; ++y) {
                                const uint32_t a[4] = {ha[2 * y], hb[2 * y], ha[2 * y + 1], hb[2 * y + 1]};
#pragma unroll
                                for (int nt = 0; nt < NT; ++nt) ptx::mma_16816<false>(acc[j][nt], a, qf[4 * j + 2 * x + y][nt]);
                            }
                        }
                    }
                }
                // S = sum_j scale_j[tok] * 2^24 * acc_j + bias_j[tok] * qsum_j ; scale/bias of both groups in one load
                float ksc[2][NG], kbi[2][NG];
#pragma unroll
                for (int ab = 0; ab < 2; ++ab) {
                    const int tok = ab ? tokB : tokA;
                    if constexpr (NG == 2) {
                        const float2 sv = h2_to_f2(*(const uint32_t*)(sbs + 0 * kTile * GROUPS + tok * 2));
                        const float2 bv = h2_to_f2(*(const uint32_t*)(sbs + 1 * kTile * GROUPS + tok * 2));
                        ksc[ab][0] = sv.x; ksc[ab][1] = sv.y; kbi[ab][0] = bv.x; kbi[ab][1] = bv.y;
                    } else {
                        ksc[ab][0] = __half2float(sbs[0 * kTile * GROUPS + tok]);
                        kbi[ab][0] = __half2float(sbs[1 * kTile * GROUPS + tok]);
                    }
                }
                const float k24 = kTwo24 * p.scale_log2e;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float v = 0.f, bq = 0.f;
#pragma unroll
                        for (int j = 0; j < NG; ++j) {
                            v = fmaf(ksc[c >> 1][j], acc[j][nt][c], v);
                            bq = fmaf(kbi[c >> 1][j], qsum[j][nt][c & 1], bq);
                        }
                        s[nt][c] = fmaf(v, k24, bq * p.scale_log2e);
                    }
            }
            if (!interior) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int tok = t0 + (c < 2 ? tokA : tokB);
                        if (tok < row_lo[nt][c & 1] || tok >= row_hi[nt][c & 1]) s[nt][c] = -INFINITY;
                    }
                if constexpr (FMT == 0) {
                    // this warp is the only reader of its 16 value rows: clear the ones past the sequence end
                    if (t0 + kTile > kv_len) {
                        const int first = max(0, kv_len - t0);
                        for (int c = lane; c < 16 * (D / 8); c += 32) {
                            const int tok = 16 * warp + c / (D / 8), ch = c % (D / 8);
                            if (tok >= first)
                                *(uint4*)(st + C::KBYTES + (ch >> 3) * (kTile * 128) + tok * 128 + (ch & 7) * 16) =
                                    make_uint4(0u, 0u, 0u, 0u);
                        }
                        ptx::fence_proxy_async();
                        __syncwarp();
                    }
                }
            }

            // ---- online softmax over this warp's tokens
            uint32_t pb[NG][NT][2];
            bool rescale = false;
            float corr[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float mx = quad_column_max(fmaxf(s[nt][e], s[nt][2 + e]));
                    const float m_new = fmaxf(m[nt][e], mx);
                    const float m_safe = m_new == -INFINITY ? 0.f : m_new;
                    corr[nt][e] = ex2(m[nt][e] - m_safe);
                    rescale |= (m_new != m[nt][e]);
                    m[nt][e] = m_new;
                    constexpr float kShift = weight_shift<FMT, BF16>();  // fp16 weights are kept away from the subnormals
                    const float pA = ex2(s[nt][e] - m_safe + kShift), pB = ex2(s[nt][2 + e] - m_safe + kShift);
                    l[nt][e] = fmaf(l[nt][e], corr[nt][e], pA + pB);
                    s[nt][e] = pA;
                    s[nt][2 + e] = pB;
                }
            if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int c = 0; c < 4; ++c) o[mt][nt][c] *= corr[nt][c & 1];
            }
            if constexpr (FMT == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    pb[0][nt][0] = movmatrix_trans(pack2<BF16>(s[nt][0], s[nt][1]));
                    pb[0][nt][1] = movmatrix_trans(pack2<BF16>(s[nt][2], s[nt][3]));
                }
            } else {
                float vsc[2][NG], vbi[2][NG];
#pragma unroll
                for (int ab = 0; ab < 2; ++ab) {
                    const int tok = ab ? tokB : tokA;
                    if constexpr (NG == 2) {
                        const float2 sv = h2_to_f2(*(const uint32_t*)(sbs + 2 * kTile * GROUPS + tok * 2));
                        const float2 bv = h2_to_f2(*(const uint32_t*)(sbs + 3 * kTile * GROUPS + tok * 2));
                        vsc[ab][0] = weight_scale(sv.x); vsc[ab][1] = weight_scale(sv.y); vbi[ab][0] = bv.x; vbi[ab][1] = bv.y;
                    } else {
                        vsc[ab][0] = weight_scale(__half2float(sbs[2 * kTile * GROUPS + tok]));
                        vbi[ab][0] = __half2float(sbs[3 * kTile * GROUPS + tok]);
                    }
                    if constexpr (FMT == 4) {
                        // the second token of a pair sits in the upper nibble and is unpacked 16 times too large
                        if (ab == 1) {
#pragma unroll
                            for (int j = 0; j < NG; ++j) vsc[ab][j] *= 0.0625f;
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < NG; ++j)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        float sc[4], bi[4];
                        if (interior) {
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                sc[c] = s[nt][c] * vsc[c >> 1][j];
                                bi[c] = s[nt][c] * vbi[c >> 1][j];
                            }
                        } else {
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                // slots past the sequence end hold stale scale/bias bytes (possibly NaN): select,
                                // never multiply them by a zero weight
                                const float pv = s[nt][c];
                                sc[c] = pv > 0.f ? pv * vsc[c >> 1][j] : 0.f;
                                bi[c] = pv > 0.f ? pv * vbi[c >> 1][j] : 0.f;
                            }
                        }
                        pb[j][nt][0] = movmatrix_trans(pack2<false>(sc[0], sc[1]));
                        pb[j][nt][1] = movmatrix_trans(pack2<false>(sc[2], sc[3]));
#pragma unroll
                        for (int e = 0; e < 2; ++e) bsum[j][nt][e] = fmaf(bsum[j][nt][e], corr[nt][e], bi[e] + bi[2 + e]);
                    }
            }

            // ---- O^T[D x rows] += V^T[D x 16 tokens] . P^T[16 tokens x rows]
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t a[4];
                const int jv = FMT == 0 ? 0 : (16 * mt) / 64;
                if constexpr (FMT == 0) {
                    ptx::ldmatrix_x4_trans(a, st_base + (mt >> 2) * (kTile * 128) + (v_off ^ (uint32_t)(((2 * mt) & 7) << 4)));
                } else if constexpr (FMT == 8) {
                    const uint32_t x = *(const uint32_t*)(st + v_off + (16 * mt) * C::VROW);
                    const uint32_t y = *(const uint32_t*)(st + v_off + (16 * mt + 8) * C::VROW);
                    a[0] = ptx::prmt(x, 0u, 0x4140u);
                    a[1] = ptx::prmt(y, 0u, 0x4140u);
                    a[2] = ptx::prmt(x, 0u, 0x4342u);
                    a[3] = ptx::prmt(y, 0u, 0x4342u);
                } else {
                    // four tokens of one element per 16-bit word: bytes to half2 positions, then the even tokens by a
                    // mask and the odd tokens (upper nibbles, 16 times too large; their weights are scaled down) by another
                    const uint32_t x = ptx::prmt((uint32_t) * (const uint16_t*)(st + v_off + (16 * mt) * C::VROW), 0u, 0x4140u);
                    const uint32_t y = ptx::prmt((uint32_t) * (const uint16_t*)(st + v_off + (16 * mt + 8) * C::VROW), 0u, 0x4140u);
                    a[0] = x & 0x000F000Fu;
                    a[1] = y & 0x000F000Fu;
                    a[2] = x & 0x00F000F0u;
                    a[3] = y & 0x00F000F0u;
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) ptx::mma_16816<(FMT == 0) && BF16>(o[mt][nt], a, pb[jv][nt]);
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty[stage]);
        }

#ifdef EMLX_TRACE_PARTS  // measurement aid: {tile loop end, part end, tiles, flags} for the first parts of a CTA
        long long trace_t0 = 0;
        if (p.trace && tid == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(trace_t0));
#endif
        // ------------------------------------------------------------------ combine the eight warps' states
        const long long a_flat = (long long)cum_u * p.Hkv + (long long)head * ntiles;
        const bool complete = (j_first == 0) && (run == ntiles);
        const int which = (max(a_flat, f_begin) != f_begin) ? 1 : 0;
        float* slot = p.slots + ((size_t)blockIdx.x * 2 + which) * kSlotFloats;
        float lw[NT][2], bw[NG][NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                lw[nt][e] = quad_column_sum(l[nt][e]);
#pragma unroll
                for (int j = 0; j < NG; ++j) bw[j][nt][e] = FMT != 0 ? quad_column_sum(bsum[j][nt][e]) : 0.f;
            }
        constexpr int PASSES = D / RC, MT_PER_PASS = RC / 16;
#pragma unroll
        for (int pass = 0; pass < PASSES; ++pass) {
            consumer_sync();  // every warp has left its tile loop / the previous pass has been read
            if (pass == 0 && g == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int row = 8 * nt + 2 * t + e;
                        wm[warp * 32 + row] = m[nt][e];
                        wl[warp * 32 + row] = lw[nt][e];
                        if constexpr (FMT != 0) {
#pragma unroll
                            for (int j = 0; j < NG; ++j) wb[(j * kConsumerWarps + warp) * 32 + row] = bw[j][nt][e];
                        }
                    }
            }
#pragma unroll
            for (int mq = 0; mq < MT_PER_PASS; ++mq) {
                const int mt = pass * MT_PER_PASS + mq;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int dl = 16 * mq + g + 8 * (c >> 1), row = 8 * nt + 2 * t + (c & 1);
                        if (row < rows_here) ored[(warp * ROWS + row) * RSTRIDE + dl] = o[mt][nt][c];
                    }
            }
            consumer_sync();
            for (int q = tid; q < rows_here * (RC / 4); q += kConsumerThreads) {  // rows past the unit's last one hold nothing
                const int row = q / (RC / 4), dl = 4 * (q - row * (RC / 4)), d = pass * RC + dl;
                float M = -INFINITY;
#pragma unroll
                for (int ww = 0; ww < kConsumerWarps; ++ww) M = fmaxf(M, wm[ww * 32 + row]);
                const float M_safe = M == -INFINITY ? 0.f : M;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                float L = 0.f, bias = 0.f;
#pragma unroll
                for (int ww = 0; ww < kConsumerWarps; ++ww) {
                    const float fw = ex2(wm[ww * 32 + row] - M_safe);
                    const float4 v = *(const float4*)(ored + (ww * ROWS + row) * RSTRIDE + dl);
                    acc.x = fmaf(fw, v.x, acc.x); acc.y = fmaf(fw, v.y, acc.y);
                    acc.z = fmaf(fw, v.z, acc.z); acc.w = fmaf(fw, v.w, acc.w);
                    L = fmaf(fw, wl[ww * 32 + row], L);
                    if constexpr (FMT != 0) bias = fmaf(fw, wb[((d / 64) * kConsumerWarps + ww) * 32 + row], bias);
                }
                if constexpr (FMT != 0) {
                    acc.x = fmaf(acc.x, kValueDown, bias); acc.y = fmaf(acc.y, kValueDown, bias);
                    acc.z = fmaf(acc.z, kValueDown, bias); acc.w = fmaf(acc.w, kValueDown, bias);
                }
                if (complete) {
                    const int r = row0 + row;
                    if (r < R) {
                        const float inv = L > 0.f ? 1.0f / L : 0.f;
                        const int i = r / p.G, hh = r - i * p.G;
                        uint2 packed;
                        packed.x = pack2<BF16>(acc.x * inv, acc.y * inv);
                        packed.y = pack2<BF16>(acc.z * inv, acc.w * inv);
                        store_out(p, out_offset<D>(p, qs + i, head * p.G + hh) + d, packed);
                    }
                } else {
                    *(float4*)(slot + row * D + d) = acc;
                    if (d == 0) {
                        slot[ROWS * D + row] = M;
                        slot[ROWS * D + ROWS + row] = L;
                    }
                }
            }
        }
        if (PEER && complete) {  // gathering call: the rows just stored go to the other ranks as well
            consumer_sync();
            peer_ready(p, peer_seen);
            peer_copy_rows<D>((uint16_t*)p.out, p.peer, p.out_Hq, p.out_head0, p.G, qs, head, row0, min(row0 + ROWS, R),
                              tid, kConsumerThreads);
        }
        if (!complete) {
            // hand the part to the merge warp: the request, then one arrival per warp after its slot stores
            if (tid == 0) {
                MergeRequest* rq = (MergeRequest*)(fixed + C::OFF_MAIL) + posted;
                rq->kind = 1; rq->row0 = row0; rq->rows = R; rq->qs = qs; rq->head = head; rq->unit = unit;
                rq->ntiles = ntiles; rq->cum_u = cum_u;
            }
            __syncwarp();
            if (lane == 0 && posted < 2) ptx::mbar_arrive(&mfull[posted]);
            ++posted;
            // a unit far longer than this CTA's slice is shared by many CTAs: worth staying for its final merge
            if (HELP && (long long)ntiles >= (kHelpMinParts - 1) * (f_end - f_begin)) may_help = true;
        }
#ifdef EMLX_TRACE_PARTS
        if (p.trace && tid == 0 && part_idx < 16) {
            long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            long long* rec = p.trace + 1024 + ((size_t)blockIdx.x * 16 + part_idx) * 4;
            rec[0] = trace_t0; rec[1] = now; rec[2] = run;
            rec[3] = (complete ? 0 : 1) | ((trace_b - trace_a) << 8) | ((trace_c - trace_b) << 24) | ((trace_d - trace_c) << 40);
        }
#endif
        remaining -= run;
        ++part_idx;
    }
    // a slice has at most two unfinished parts (its first and its last); tell the merge warp that no more follow
    for (; posted < 2; ++posted) {
        if (tid == 0) ((MergeRequest*)(fixed + C::OFF_MAIL))[posted].kind = 2;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&mfull[posted]);
    }
    if constexpr (HELP) {
        if (may_help) park_consumer_warp<D, NT, FMT, BF16, PEER>(p, fixed, full, abort_word);
    }
}

// ---- the final merge of a unit, shared by the consumer warps --------------------------------------------------
// A unit that is split over many CTAs (a few long sequences on the whole GPU) ends with one warp folding all its
// parts: every part costs a round trip to L2 and a warp can keep only a few kilobytes in flight, so eighteen parts
// took about 16 us at the very end of the kernel.  Consumer warps that have finished their slice therefore park
// instead of leaving; when the merge warp finds all eight parked it computes the weights of the parts, writes them
// and the parts' addresses to shared memory and lets every warp fold one or two rows with all its loads in flight.
// The arithmetic (weights, order of the parts, denominators) is that of the one-warp path, so the result does not
// depend on which path a launch happened to take.
template <int ROWS>
struct MergeJob {
    int nparts, rows_here, pad0, pad1;
    MergeRequest rq;
    float den[16];
    unsigned long long slot[kHelpParts];  // partial rows of part j (0: that slice holds no tiles)
    float w[kHelpParts][ROWS];            // weight of part j for row r
    float l[kHelpParts][ROWS];            // sum of part j for row r
};

template <int D, int NT, int FMT, bool BF16, bool PEER>
__device__ __forceinline__ void help_merge(const TiledParams& p, const MergeJob<Cfg<D, NT, FMT>::ROWS>* job, int warp, int lane) {
    constexpr int ROWS = Cfg<D, NT, FMT>::ROWS, V = D / 32, B = 8;
    const int nparts = job->nparts;
    const MergeRequest rq = job->rq;
    for (int row = warp; row < ROWS; row += kConsumerWarps) {
        const int r = rq.row0 + row;
        if (r >= rq.rows) continue;
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] = 0.f;
        for (int j0 = 0; j0 < nparts; j0 += B) {
            float wr[B], v[B][V];
#pragma unroll
            for (int u = 0; u < B; ++u) {
                const int j = j0 + u;
                const float* sl = j < nparts ? (const float*)job->slot[j] : nullptr;
                wr[u] = sl ? job->w[j][row] : 0.f;
                if constexpr (V == 4) {
                    const float4 x = sl ? __ldcg((const float4*)(sl + row * D) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
                    v[u][0] = x.x; v[u][1] = x.y; v[u][2] = x.z; v[u][3] = x.w;
                } else {
                    const float2 x = sl ? __ldcg((const float2*)(sl + row * D) + lane) : make_float2(0.f, 0.f);
                    v[u][0] = x.x; v[u][1] = x.y;
                }
            }
#pragma unroll
            for (int u = 0; u < B; ++u)
                if (wr[u] != 0.f) {
#pragma unroll
                    for (int k = 0; k < V; ++k) acc[k] = fmaf(wr[u], v[u][k], acc[k]);
                }
        }
        const float dr = job->den[row];
        const int i = r / p.G, hh = r - i * p.G;
        const long long dst = out_offset<D>(p, rq.qs + i, rq.head * p.G + hh) + V * lane;
        float o[V];
#pragma unroll
        for (int k = 0; k < V; ++k) o[k] = dr > 0.f ? acc[k] / dr : 0.f;
        if constexpr (V == 4) {
            uint2 packed;
            packed.x = pack2<BF16>(o[0], o[1]);
            packed.y = pack2<BF16>(o[2], o[3]);
            store_out(p, dst, packed);
        } else {
            store_out(p, dst, pack2<BF16>(o[0], o[1]));
        }
        if constexpr (PEER) {  // the merge warp has seen the other ranks' ready flags before it handed out the job
            __syncwarp();
            peer_copy_rows<D>((uint16_t*)p.out, p.peer, p.out_Hq, p.out_head0, p.G, rq.qs, rq.head, r, r + 1, lane, 32);
        }
    }
}

// Consumer warps that have finished their slice: wait for jobs of the merge warp until it says that it has left.
template <int D, int NT, int FMT, bool BF16, bool PEER>
__device__ __forceinline__ void park_consumer_warp(const TiledParams& p, uint8_t* fixed, uint64_t* full,
                                                   volatile int* abort_word) {
    using C = Cfg<D, NT, FMT>;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t *parked = full + 26, *go = full + 27, *done = full + 28;
    volatile int* misc = (volatile int*)(fixed + C::OFF_MISC);
    if (*abort_word) return;
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(parked);
    for (uint32_t job_idx = 0;; ++job_idx) {
        int ok = 0;
        if (lane == 0) {
            for (uint32_t i = 0; i < (1u << 22) && !ok && !*abort_word; ++i) {
                ok = ptx::mbar_try_wait(go, job_idx & 1) ? 1 : 0;
                if (!ok) __nanosleep(i < 4096 ? 32 : 500);
            }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
            if (!*abort_word) *abort_word = 1;
            return;
        }
        if (misc[kMiscHelpExit]) return;
        help_merge<D, NT, FMT, BF16, PEER>(p, (const MergeJob<C::ROWS>*)(fixed + C::PBYTES), warp, lane);
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(done);
    }
}

// The merge warp.  For every unfinished part the consumers hand over: make the slot visible to the GPU, count the
// arrival on the (unit, head) counter, and when this was the last of the unit's parts, fold all of them in slice
// order (so the result does not depend on which CTA came last) and write the rows.
template <int D, int NT, int FMT, bool BF16, bool PEER, bool HELP>
__device__ __forceinline__ void merge_warp_loop(const TiledParams& p, uint8_t* fixed, uint64_t* full,
                                                volatile int* abort_word, int active) {
    using C = Cfg<D, NT, FMT>;
    constexpr int ROWS = C::ROWS;
    const int lane = threadIdx.x & 31;
    uint64_t* mfull = full + 24;
    bool peer_seen = false;
    uint32_t jobs_posted = 0;  // final merges handed to the parked consumer warps
    if constexpr (PEER) peer_ready(p, peer_seen);  // while the consumers work: off the path of the merge
    for (int e = 0; e < 2; ++e) {
        // the consumers may take their whole slice before they post: sleep between polls, give up after seconds
        int ok = 0;
        if (lane == 0) {
            for (uint32_t i = 0; i < (1u << 22) && !ok && !*abort_word; ++i) {
                ok = ptx::mbar_try_wait(&mfull[e], 0) ? 1 : 0;
                if (!ok) __nanosleep(i < 64 ? 200 : 2000);
            }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);  // one decision for the warp; the shuffle also orders the lanes' reads
        if (!ok) {
            if (!*abort_word) *abort_word = 1;
            if (lane == 0) flag_error(p.status, EMLX_DEV_WAIT_TIMEOUT);
            return;
        }
        const MergeRequest rq = ((const MergeRequest*)(fixed + C::OFF_MAIL))[e];
        if (rq.kind != 1) return;
        const long long a_flat = (long long)rq.cum_u * p.Hkv + (long long)rq.head * rq.ntiles;
        const long long b_flat = a_flat + rq.ntiles;
        const int c_first = warp_last_true(0, active, lane, [&](int c) { return p.cta_start[c] <= a_flat; });
        const int c_last = warp_last_true(0, active, lane, [&](int c) { return p.cta_start[c] <= b_flat - 1; });
        const int nparts = slices_in_use(p.cta_start, c_first, c_last);
        int* counter = p.counters + (size_t)rq.unit * p.Hkv + rq.head;
        __threadfence();  // the consumers' slot stores, seen through the barrier, become visible GPU-wide
        int ticket = 0;
        if (lane == 0) ticket = atomicAdd(counter, 1);
        ticket = __shfl_sync(0xffffffffu, ticket, 0);
        if (ticket != nparts - 1) continue;
        __threadfence();
#ifdef EMLX_TRACE_TIMELINE
        if (p.trace && lane == 0) {
            long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            p.trace[2048 + 4 * blockIdx.x + 2] = now;
        }
#endif
        const int span = c_last - c_first + 1;
        int all_parked = 0;
        if (HELP && span >= kHelpMinParts && span <= kHelpParts) {
            if (lane == 0) all_parked = ptx::mbar_try_wait(full + 26, 0) ? 1 : 0;
            all_parked = __shfl_sync(0xffffffffu, all_parked, 0);
        }
        if (HELP && all_parked) {
            // the consumer warps fold the rows; this warp prepares what they need (lane j looks at part base + j)
            MergeJob<ROWS>* job = (MergeJob<ROWS>*)(fixed + C::PBYTES);
            static_assert(sizeof(MergeJob<ROWS>) <= (size_t)C::OREDBYTES, "the job does not fit the reduction scratch");
            float Mr[ROWS];
#pragma unroll
            for (int row = 0; row < ROWS; ++row) Mr[row] = -INFINITY;
            for (int base = 0; base < span; base += 32) {
                const int c = c_first + base + lane;
                unsigned long long mine = 0;
                if (c <= c_last) {
                    const long long cb = p.cta_start[c];
                    if (cb < p.cta_start[c + 1])
                        mine = (unsigned long long)(p.slots + ((size_t)c * 2 + (max(a_flat, cb) != cb ? 1 : 0)) * kSlotFloats);
                    job->slot[base + lane] = mine;
                }
                const float* sl = (const float*)mine;
                float mp[ROWS], lp[ROWS];
#pragma unroll
                for (int row = 0; row < ROWS; ++row) {
                    mp[row] = sl ? __ldcg(sl + ROWS * D + row) : -INFINITY;
                    lp[row] = sl ? __ldcg(sl + ROWS * D + ROWS + row) : 0.f;
                }
#pragma unroll
                for (int row = 0; row < ROWS; ++row) {
                    Mr[row] = fmaxf(Mr[row], warp_max(lp[row] > 0.f ? mp[row] : -INFINITY));
                    if (c <= c_last) {
                        job->w[base + lane][row] = mp[row];  // the maximum for now; the weight once M is known
                        job->l[base + lane][row] = lp[row];
                    }
                }
            }
            __syncwarp();
            for (int j = lane; j < span; j += 32)
#pragma unroll
                for (int row = 0; row < ROWS; ++row) {
                    const float lp = job->l[j][row];
                    job->w[j][row] = lp > 0.f ? ex2(job->w[j][row] - Mr[row]) : 0.f;
                }
            __syncwarp();
            if (lane < ROWS) {
                float den = 0.f;
                for (int j = 0; j < span; ++j)
                    if (job->slot[j]) den = fmaf(job->w[j][lane], job->l[j][lane], den);
                job->den[lane] = den;
            }
            if (lane == 0) {
                job->nparts = span;
                job->rows_here = min(ROWS, rq.rows - rq.row0);
                job->rq = rq;
            }
            __syncwarp();
            int ok = 0;
            if (lane == 0) {
                ptx::mbar_arrive(full + 27);
                for (uint32_t i = 0; i < (1u << 22) && !ok && !*abort_word; ++i) {
                    ok = ptx::mbar_try_wait(full + 28, jobs_posted & 1) ? 1 : 0;
                    if (!ok) __nanosleep(i < 256 ? 50 : 2000);
                }
            }
            ++jobs_posted;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (!*abort_word) *abort_word = 1;
                if (lane == 0) flag_error(p.status, EMLX_DEV_WAIT_TIMEOUT);
                return;
            }
            if (lane == 0) *counter = 0;
            continue;
        }
        // Lane r < ROWS folds the parts' (max, sum) pairs of row r; lane l folds head_dim elements [V*l, V*l + V) of
        // every row: one vector load per row and part, one vector store per row.
        const int rows_here = min(ROWS, rq.rows - rq.row0);
        const int lrow = lane < ROWS ? lane : 0;
        constexpr int V = D / 32;
        float acc[ROWS][V], den = 0.f, M = -INFINITY;
#pragma unroll
        for (int row = 0; row < ROWS; ++row)
#pragma unroll
            for (int k = 0; k < V; ++k) acc[row][k] = 0.f;
        auto load_rows = [&](const float* sl, float (&v)[ROWS][V]) {
#pragma unroll
            for (int row = 0; row < ROWS; ++row) {
                if constexpr (V == 4) {
                    const float4 x = (sl && row < rows_here) ? __ldcg((const float4*)(sl + row * D) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
                    v[row][0] = x.x; v[row][1] = x.y; v[row][2] = x.z; v[row][3] = x.w;
                } else {
                    const float2 x = (sl && row < rows_here) ? __ldcg((const float2*)(sl + row * D) + lane) : make_float2(0.f, 0.f);
                    v[row][0] = x.x; v[row][1] = x.y;
                }
            }
        };
        auto fold = [&](float wgt, const float (&v)[ROWS][V]) {
#pragma unroll
            for (int row = 0; row < ROWS; ++row) {
                const float wr = __shfl_sync(0xffffffffu, wgt, row);
                if (wr != 0.f) {
#pragma unroll
                    for (int k = 0; k < V; ++k) acc[row][k] = fmaf(wr, v[row][k], acc[row][k]);
                }
            }
        };
        {
            for (int c = c_first; c <= c_last; ++c) {
                const long long cb = p.cta_start[c];
                if (cb >= p.cta_start[c + 1]) continue;
                const float* sl = p.slots + ((size_t)c * 2 + (max(a_flat, cb) != cb ? 1 : 0)) * kSlotFloats;
                const float mp = __ldcg(sl + ROWS * D + lrow), lp = __ldcg(sl + ROWS * D + ROWS + lrow);
                if (lp > 0.f) M = fmaxf(M, mp);
            }
#pragma unroll 1
            for (int c = c_first; c <= c_last; ++c) {
                const long long cb = p.cta_start[c];
                if (cb >= p.cta_start[c + 1]) continue;
                const float* sl = p.slots + ((size_t)c * 2 + (max(a_flat, cb) != cb ? 1 : 0)) * kSlotFloats;
                const float mp = __ldcg(sl + ROWS * D + lrow), lp = __ldcg(sl + ROWS * D + ROWS + lrow);
                const float wgt = lp > 0.f ? ex2(mp - M) : 0.f;
                den = fmaf(wgt, lp, den);
                float v[ROWS][V];
                load_rows(sl, v);
                fold(wgt, v);
            }
        }
#pragma unroll
        for (int row = 0; row < ROWS; ++row) {
            const float dr = __shfl_sync(0xffffffffu, den, row);
            const int r = rq.row0 + row;
            if (r < rq.rows) {
                const int i = r / p.G, hh = r - i * p.G;
                const long long dst = out_offset<D>(p, rq.qs + i, rq.head * p.G + hh) + V * lane;
                float o[V];
#pragma unroll
                for (int k = 0; k < V; ++k) o[k] = dr > 0.f ? acc[row][k] / dr : 0.f;
                if constexpr (V == 4) {
                    uint2 packed;
                    packed.x = pack2<BF16>(o[0], o[1]);
                    packed.y = pack2<BF16>(o[2], o[3]);
                    store_out(p, dst, packed);
                } else {
                    store_out(p, dst, pack2<BF16>(o[0], o[1]));
                }
            }
        }
        if constexpr (PEER) {
            __syncwarp();
            peer_copy_rows<D>((uint16_t*)p.out, p.peer, p.out_Hq, p.out_head0, p.G, rq.qs, rq.head, rq.row0,
                              min(rq.row0 + ROWS, rq.rows), lane, 32);
        }
        if (lane == 0) *counter = 0;
#ifdef EMLX_TRACE_TIMELINE
        if (p.trace && lane == 0) {
            long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            p.trace[2048 + 4 * blockIdx.x + 3] = now;
        }
#endif
    }
}

}  // namespace emlx
