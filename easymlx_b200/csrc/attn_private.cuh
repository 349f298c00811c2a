// Consumer loop for units of up to 16 query rows (decode, small GQA groups): every consumer warp owns 16
// tokens of each 128-token tile from score to output accumulation, with its own running max / sum and its
// own O^T[D x rows] accumulators, so consumer warps never meet at a barrier inside the tile loop and drift
// apart to hide each other's latencies.  The eight partial states are combined once per (unit, head) part.
// Included by attn_tiled.cu after Cfg, TiledParams, Walk and the small helpers.
#pragma once

namespace emlx {

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
template <bool BF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    return (uint32_t)to_bits16<BF16>(lo) | ((uint32_t)to_bits16<BF16>(hi) << 16);
}

template <int D, int NT, int FMT, bool BF16>
__device__ __forceinline__ void consumer_loop_private(const TiledParams& p, uint8_t* stages, uint8_t* fixed,
                                                      uint64_t* full, uint64_t* empty, volatile int* abort_word,
                                                      long long f_begin, long long f_end, int num_units,
                                                      long long total_flat, long long active) {
    using C = Cfg<D, NT, FMT>;
    constexpr int KS = D / 16, MT = D / 16, ROWS = C::ROWS, GROUPS = C::GROUPS;
    constexpr int NG = FMT == 0 ? 1 : GROUPS;
    constexpr int HALVES = D / 64;  // the cross-warp reduction goes through shared memory 64 columns of D at a time
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    uint8_t* stage_out = fixed;                       // [ROWS][D*2 + 16] output rows before the coalesced store
    float* ored = (float*)(fixed + C::PBYTES);        // [warps][64][ROWS]
    float* rowM = (float*)(fixed + C::PBYTES + C::OREDBYTES);  // [32] merged max, then [32] merged sum
    float* rowL = rowM + 32;
    float* wm = rowL + 32;                            // [warps][32] per-warp running max
    float* wl = wm + kConsumerWarps * 32;             // [warps][32] per-warp running sum
    float* wb = wl + kConsumerWarps * 32;             // [2][warps][32] per-warp bias terms of the values
    int* misc = (int*)(wb + 2 * kConsumerWarps * 32);
    constexpr int OUT_STRIDE = D * 2 + 16;

    // token of the tile that MMA row g (and g + 8) of this warp stands for; the affine formats permute
    // tokens so that the transposed probabilities line up with the way value codes are unpacked
    const int tokA = 16 * warp + (FMT == 0 ? g : (FMT == 8 ? 4 * (g >> 1) + (g & 1) : 4 * (g >> 1) + 2 * (g & 1)));
    const int tokB = tokA + (FMT == 0 ? 8 : (FMT == 8 ? 2 : 1));

    Walk w;
    w.locate(f_begin, p.unit_cum, num_units, p.Hkv);
    long long f = f_begin;
    uint32_t it = 0;

    while (f < f_end) {
        const int seq = p.unit_seq[w.u], row0 = p.unit_row0[w.u], tile_lo = p.unit_tile_lo[w.u];
        const int qs = p.qsl[seq], q_len = p.qsl[seq + 1] - qs, kv_len = p.kv_lens[seq];
        const int R = q_len * p.G, ctx = kv_len - q_len, head = w.head;
        const int run = (int)min((long long)(w.ntiles - w.j), f_end - f);
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

        uint32_t qf[KS][NT][2];
        float qsum[NG][NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int r = row0 + 8 * nt + g;
            const bool ok = r < R;
            const int i = ok ? r / p.G : 0, hh = ok ? r - i * p.G : 0;
            const uint16_t* qrow = (const uint16_t*)p.q + ((long long)(qs + i) * p.Hq + head * p.G + hh) * D;
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
#pragma unroll
                for (int jx = 0; jx < KS / 2; ++jx) {
                    const uint4 v = ok ? *(const uint4*)(qrow + 64 * (jx >> 1) + 16 * t + 8 * (jx & 1)) : make_uint4(0u, 0u, 0u, 0u);
                    qf[2 * jx][nt][0] = ptx::prmt(v.x, v.y, 0x5410u);
                    qf[2 * jx][nt][1] = ptx::prmt(v.z, v.w, 0x5410u);
                    qf[2 * jx + 1][nt][0] = ptx::prmt(v.x, v.y, 0x7632u);
                    qf[2 * jx + 1][nt][1] = ptx::prmt(v.z, v.w, 0x7632u);
                }
            }
        }
        if constexpr (FMT != 0) {
            const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};
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

        for (int jj = 0; jj < run; ++jj, ++it) {
            const uint32_t stage = it % C::STAGES;
            uint8_t* st = stages + (size_t)stage * C::STAGE;
            const uint32_t ks_base = ptx::smem_u32(st), vs_base = ks_base + C::KBYTES;
            const __half* sbs = (const __half*)(st + C::KBYTES + C::VBYTES);
            const int t0 = (tile_lo + w.j + jj) * kTile;
            const bool interior = (t0 + kTile <= hi_min) && (t0 >= lo_max);
            ptx::mbar_wait(&full[stage], (it / C::STAGES) & 1, abort_word);

            // ---- scores of this warp's 16 tokens against every row
            float s[NT][4];
            if constexpr (FMT == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const uint32_t off = (uint32_t)((ks >> 2) * (kTile * 128) + (16 * warp + (lane & 15)) * 128 +
                                                    ((ks & 3) * 2 + (lane >> 4)) * 16);
                    uint32_t a[4];
                    ptx::ldmatrix_x4(a, ks_base + ptx::swz<3>(off));
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
                        const uint4 xa = *(const uint4*)(st + ptx::swz<C::KSW>((uint32_t)(tokA * C::KROW + 64 * j + 16 * t)));
                        const uint4 xb = *(const uint4*)(st + ptx::swz<C::KSW>((uint32_t)(tokB * C::KROW + 64 * j + 16 * t)));
                        const uint32_t wa[4] = {xa.x, xa.y, xa.z, xa.w}, wbv[4] = {xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                        for (int sidx = 0; sidx < 4; ++sidx) {
                            const uint32_t a[4] = {ptx::prmt(wa[sidx], 0u, 0x4140u), ptx::prmt(wbv[sidx], 0u, 0x4140u),
                                                   ptx::prmt(wa[sidx], 0u, 0x4342u), ptx::prmt(wbv[sidx], 0u, 0x4342u)};
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) ptx::mma_16816<false>(acc[j][nt], a, qf[4 * j + sidx][nt]);
                        }
                    } else {
                        const uint2 xa = *(const uint2*)(st + ptx::swz<C::KSW>((uint32_t)(tokA * C::KROW + 32 * j + 8 * t)));
                        const uint2 xb = *(const uint2*)(st + ptx::swz<C::KSW>((uint32_t)(tokB * C::KROW + 32 * j + 8 * t)));
                        const uint32_t wa[2] = {xa.x, xa.y}, wbv[2] = {xb.x, xb.y};
#pragma unroll
                        for (int x = 0; x < 2; ++x) {
                            uint32_t ha[4], hb[4];
                            nibbles_to_h2(wa[x], ha);
                            nibbles_to_h2(wbv[x], hb);
#pragma unroll
                            for (int y = 0; y < 2; ++y) {
                                const uint32_t a[4] = {ha[2 * y], hb[2 * y], ha[2 * y + 1], hb[2 * y + 1]};
#pragma unroll
                                for (int nt = 0; nt < NT; ++nt) ptx::mma_16816<false>(acc[j][nt], a, qf[4 * j + 2 * x + y][nt]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int tok = c < 2 ? tokA : tokB;
                        float v = 0.f;
#pragma unroll
                        for (int j = 0; j < NG; ++j)
                            v += __half2float(sbs[0 * kTile * GROUPS + tok * GROUPS + j]) * kTwo24 * acc[j][nt][c] +
                                 __half2float(sbs[1 * kTile * GROUPS + tok * GROUPS + j]) * qsum[j][nt][c & 1];
                        s[nt][c] = v * p.scale_log2e;
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
                    corr[nt][e] = exp2f(m[nt][e] - m_safe);
                    rescale |= (m_new != m[nt][e]);
                    m[nt][e] = m_new;
                    const float pA = exp2f(s[nt][e] - m_safe), pB = exp2f(s[nt][2 + e] - m_safe);
                    l[nt][e] = l[nt][e] * corr[nt][e] + pA + pB;
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
#pragma unroll
                for (int j = 0; j < NG; ++j) {
                    const float vsA = __half2float(sbs[2 * kTile * GROUPS + tokA * GROUPS + j]);
                    const float vsB = __half2float(sbs[2 * kTile * GROUPS + tokB * GROUPS + j]);
                    const float vbA = __half2float(sbs[3 * kTile * GROUPS + tokA * GROUPS + j]);
                    const float vbB = __half2float(sbs[3 * kTile * GROUPS + tokB * GROUPS + j]);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        float sc[4], bi[4];
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            // stale scale/bias of unwritten slots may be NaN: select, never multiply by a zero weight
                            const float pv = s[nt][c];
                            sc[c] = pv > 0.f ? pv * (c < 2 ? vsA : vsB) : 0.f;
                            bi[c] = pv > 0.f ? pv * (c < 2 ? vbA : vbB) : 0.f;
                        }
                        pb[j][nt][0] = movmatrix_trans(pack2<false>(sc[0], sc[1]));
                        pb[j][nt][1] = movmatrix_trans(pack2<false>(sc[2], sc[3]));
#pragma unroll
                        for (int e = 0; e < 2; ++e) bsum[j][nt][e] = bsum[j][nt][e] * corr[nt][e] + bi[e] + bi[2 + e];
                    }
                }
            }

            // ---- O^T[D x rows] += V^T[D x 16 tokens] . P^T[16 tokens x rows]
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t a[4];
                const int jv = FMT == 0 ? 0 : (16 * mt) / 64;
                if constexpr (FMT == 0) {
                    const int tok = 16 * warp + (lane & 7) + 8 * (lane >> 4);
                    const int ch = 2 * mt + ((lane >> 3) & 1);
                    ptx::ldmatrix_x4_trans(a, vs_base + ptx::swz<3>((uint32_t)((ch >> 3) * (kTile * 128) + tok * 128 + (ch & 7) * 16)));
                } else if constexpr (FMT == 8) {
                    const uint32_t x = *(const uint32_t*)(st + C::KBYTES + ptx::swz<C::VSW>((uint32_t)((16 * mt + g) * C::VROW + 16 * warp + 4 * t)));
                    const uint32_t y = *(const uint32_t*)(st + C::KBYTES + ptx::swz<C::VSW>((uint32_t)((16 * mt + g + 8) * C::VROW + 16 * warp + 4 * t)));
                    a[0] = ptx::prmt(x, 0u, 0x4140u);
                    a[1] = ptx::prmt(y, 0u, 0x4140u);
                    a[2] = ptx::prmt(x, 0u, 0x4342u);
                    a[3] = ptx::prmt(y, 0u, 0x4342u);
                } else {
                    const uint32_t x = *(const uint16_t*)(st + C::KBYTES + ptx::swz<C::VSW>((uint32_t)((16 * mt + g) * C::VROW + 8 * warp + 2 * t)));
                    const uint32_t y = *(const uint16_t*)(st + C::KBYTES + ptx::swz<C::VSW>((uint32_t)((16 * mt + g + 8) * C::VROW + 8 * warp + 2 * t)));
                    const uint32_t z = x | (y << 16);
                    const uint32_t lo = z & 0x0F0F0F0Fu, hi = (z >> 4) & 0x0F0F0F0Fu;
                    a[0] = ptx::prmt(lo, 0u, 0x4140u);
                    a[1] = ptx::prmt(lo, 0u, 0x4342u);
                    a[2] = ptx::prmt(hi, 0u, 0x4140u);
                    a[3] = ptx::prmt(hi, 0u, 0x4342u);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) ptx::mma_16816<(FMT == 0) && BF16>(o[mt][nt], a, pb[jv][nt]);
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty[stage]);
        }

        // ------------------------------------------------------------------ combine the eight warps' states
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float lw = quad_column_sum(l[nt][e]);
                if (g == 0) {
                    wm[warp * 32 + 8 * nt + 2 * t + e] = m[nt][e];
                    wl[warp * 32 + 8 * nt + 2 * t + e] = lw;
                }
                if constexpr (FMT != 0) {
#pragma unroll
                    for (int j = 0; j < NG; ++j) {
                        const float bw = quad_column_sum(bsum[j][nt][e]);
                        if (g == 0) wb[(j * kConsumerWarps + warp) * 32 + 8 * nt + 2 * t + e] = bw;
                    }
                }
            }
        consumer_sync();
        float fac[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int row = 8 * nt + 2 * t + e;
                float M = -INFINITY;
#pragma unroll
                for (int ww = 0; ww < kConsumerWarps; ++ww) M = fmaxf(M, wm[ww * 32 + row]);
                const float M_safe = M == -INFINITY ? 0.f : M;
                float L = 0.f;
#pragma unroll
                for (int ww = 0; ww < kConsumerWarps; ++ww) {
                    const float fw = exp2f(wm[ww * 32 + row] - M_safe);
                    L += fw * wl[ww * 32 + row];
                }
                fac[nt][e] = exp2f(m[nt][e] - M_safe) * (FMT != 0 ? kTwo24 : 1.0f);
                if (warp == 0 && g == 0) {
                    rowM[row] = M;
                    rowL[row] = L;
                }
            }

        const long long a_flat = (long long)p.unit_cum[w.u] * p.Hkv + (long long)head * w.ntiles;
        const long long b_flat = a_flat + w.ntiles;
        const bool complete = (w.j == 0) && (run == w.ntiles);
        const long long P = active;
        const int which = (max(a_flat, f_begin) != f_begin) ? 1 : 0;
        float* slot = p.slots + ((size_t)blockIdx.x * 2 + which) * kSlotFloats;

        // sum of the scaled accumulators over warps, 64 columns of D at a time, in warp order
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
            if (h > 0) consumer_sync();  // the previous half has been read
#pragma unroll
            for (int mq = 0; mq < 4; ++mq) {
                const int mt = 4 * h + mq;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int dl = 16 * mq + g + 8 * (c >> 1), row = 8 * nt + 2 * t + (c & 1);
                        ored[(warp * 64 + dl) * ROWS + row] = o[mt][nt][c] * fac[nt][c & 1];
                    }
            }
            consumer_sync();
            for (int idx = tid; idx < 64 * ROWS; idx += kConsumerThreads) {
                const int dl = idx / ROWS, row = idx - dl * ROWS, d = 64 * h + dl;
                float v = 0.f;
#pragma unroll
                for (int ww = 0; ww < kConsumerWarps; ++ww) v += ored[(ww * 64 + dl) * ROWS + row];
                if constexpr (FMT != 0) {
                    // bias term of this column's scale group: sum_w f_w * sum_tok P * vb
                    float bt = 0.f;
                    const float M = rowM[row], M_safe = M == -INFINITY ? 0.f : M;
#pragma unroll
                    for (int ww = 0; ww < kConsumerWarps; ++ww)
                        bt += exp2f(wm[ww * 32 + row] - M_safe) * wb[((d / 64) * kConsumerWarps + ww) * 32 + row];
                    v += bt;
                }
                if (complete) {
                    const float L = rowL[row];
                    *(uint16_t*)(stage_out + row * OUT_STRIDE + d * 2) = to_bits16<BF16>(L > 0.f ? v / L : 0.f);
                } else {
                    slot[row * D + d] = v;
                }
            }
        }
        if (complete) {
            consumer_sync();
            constexpr int CH = D / 8;
            for (int idx = tid; idx < ROWS * CH; idx += kConsumerThreads) {
                const int row = idx / CH, ch = idx - row * CH, r = row0 + row;
                if (r < R) {
                    const int i = r / p.G, hh = r - i * p.G;
                    uint16_t* dst = (uint16_t*)p.out + ((long long)(qs + i) * p.Hq + head * p.G + hh) * D + ch * 8;
                    *(uint4*)dst = *(const uint4*)(stage_out + row * OUT_STRIDE + ch * 16);
                }
            }
        } else {
            if (tid < ROWS) {
                slot[ROWS * D + tid] = rowM[tid];
                slot[ROWS * D + ROWS + tid] = rowL[tid];
            }
            __threadfence();
            consumer_sync();
            const int c_first = (int)(((a_flat + 1) * P - 1) / total_flat);
            const int c_last = (int)((b_flat * P - 1) / total_flat);
            int* counter = p.counters + (size_t)w.u * p.Hkv + head;
            if (tid == 0) misc[1] = atomicAdd(counter, 1);
            consumer_sync();
            if (misc[1] == c_last - c_first) {
                __threadfence();
                for (int idx = tid; idx < ROWS * D; idx += kConsumerThreads) {
                    const int row = idx / D, d = idx - row * D, r = row0 + row;
                    if (r >= R) continue;
                    float M = -INFINITY;
                    for (int c = c_first; c <= c_last; ++c) {
                        const long long cb = total_flat * c / P;
                        const float* sl = p.slots + ((size_t)c * 2 + (max(a_flat, cb) != cb ? 1 : 0)) * kSlotFloats;
                        if (__ldcg(sl + ROWS * D + ROWS + row) > 0.f) M = fmaxf(M, __ldcg(sl + ROWS * D + row));
                    }
                    float acc = 0.f, den = 0.f;
                    for (int c = c_first; c <= c_last; ++c) {
                        const long long cb = total_flat * c / P;
                        const float* sl = p.slots + ((size_t)c * 2 + (max(a_flat, cb) != cb ? 1 : 0)) * kSlotFloats;
                        const float lp = __ldcg(sl + ROWS * D + ROWS + row);
                        if (lp > 0.f) {
                            const float wgt = exp2f(__ldcg(sl + ROWS * D + row) - M);
                            acc += wgt * __ldcg(sl + row * D + d);
                            den += wgt * lp;
                        }
                    }
                    const int i = r / p.G, hh = r - i * p.G;
                    ((uint16_t*)p.out)[((long long)(qs + i) * p.Hq + head * p.G + hh) * D + d] =
                        to_bits16<BF16>(den > 0.f ? acc / den : 0.f);
                }
                if (tid == 0) *counter = 0;
            }
        }
        consumer_sync();
        f += run;
        w.next_part(p.unit_cum, num_units, p.Hkv);
    }
}

}  // namespace emlx
