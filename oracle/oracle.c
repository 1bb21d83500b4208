/* TEST INFRASTRUCTURE ONLY - see oracle.h.  Scalar C restatement of the
 * reference's CPU integer GEMV/GEMM arithmetic from raw GGUF blocks.
 * Build: gcc -std=c11 -O2 -ffp-contract=off -pthread (see Makefile).
 */
#include "oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ---------------------------------------------------------------- parallel for
 * Static split of [0, n) over ORC_THREADS (default: online CPUs) pthreads.  Each
 * index is computed independently, so the thread count never changes a result. */
typedef void (*par_fn)(int i, void * ctx);
typedef struct {
    par_fn fn;
    void * ctx;
    int lo, hi;
} par_job;

static void * par_main(void * p) {
    par_job * j = (par_job *)p;
    for (int i = j->lo; i < j->hi; i++) {
        j->fn(i, j->ctx);
    }
    return NULL;
}

static int par_threads(void) {
    const char * e = getenv("ORC_THREADS");
    int n = e ? atoi(e) : (int)sysconf(_SC_NPROCESSORS_ONLN);
    return n < 1 ? 1 : (n > 256 ? 256 : n);
}

static void par_for(int n, par_fn fn, void * ctx) {
    int nt = par_threads();
    if (nt > n) {
        nt = n;
    }
    if (nt <= 1) {
        par_job j = {fn, ctx, 0, n};
        par_main(&j);
        return;
    }
    pthread_t th[256];
    par_job jobs[256];
    for (int k = 0; k < nt; k++) {
        jobs[k].fn = fn;
        jobs[k].ctx = ctx;
        jobs[k].lo = (int)((long long)n * k / nt);
        jobs[k].hi = (int)((long long)n * (k + 1) / nt);
        pthread_create(&th[k], NULL, par_main, &jobs[k]);
    }
    for (int k = 0; k < nt; k++) {
        pthread_join(th[k], NULL);
    }
}

/* ------------------------------------------------------------------ f16 <-> f32
 * Follows src/common/quant.h:67-133 of the reference: the f32->f16 direction
 * TRUNCATES the mantissa (no rounding), produces f16 subnormals by shifting the
 * 24-bit significand, and maps every overflow (and NaN) to +-inf. */
float orc_h2f(uint16_t h) {
    const uint32_t s = (uint32_t)(h >> 15) << 31;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, bits;
    if (e == 0) {
        if (m == 0) {
            bits = s;
        } else {
            int ex = 127 - 15 + 1;
            while (!(m & 0x400u)) {
                m <<= 1;
                ex--;
            }
            bits = s | ((uint32_t)ex << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (e == 31) {
        bits = s | 0x7F800000u | (m << 13);
    } else {
        bits = s | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t orc_f2h(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    const uint32_t s = (bits >> 16) & 0x8000u;
    const int32_t e32 = (int32_t)((bits >> 23) & 0xFF);
    const int32_t e16 = e32 - 112;
    const uint32_t m = bits & 0x7FFFFFu;
    if (e16 >= 31) {
        return (uint16_t)(s | 0x7C00u);
    }
    if (e16 <= 0) {
        const int32_t sh = 126 - e32;
        if (sh >= 32) {
            return (uint16_t)s;
        }
        return (uint16_t)(s | ((m | 0x800000u) >> sh));
    }
    return (uint16_t)(s | ((uint32_t)e16 << 10) | (m >> 13));
}

/* ---------------------------------------------------------------- block geometry
 * src/common/quant.h:12-41, 292-298, 1177-1198 */
enum { SB_Q4K = 144, SB_Q5K = 176, SB_Q6K = 210, SB_IQ4XS = 136, B_Q80 = 34 };

size_t orc_row_bytes(uint32_t type, int64_t n) {
    switch (type) {
    case ORC_Q4_K: return (size_t)(n / 256) * SB_Q4K;
    case ORC_Q5_K: return (size_t)(n / 256) * SB_Q5K;
    case ORC_Q6_K: return (size_t)(n / 256) * SB_Q6K;
    case ORC_IQ4_XS: return (size_t)(n / 256) * SB_IQ4XS;
    case ORC_Q8_0: return (size_t)(n / 32) * B_Q80;
    default: return 0;
    }
}

/* number of int32 partial dots a row produces: one per 32-value group, except
 * Q6_K whose scale groups hold 16 values (src/backend/cpu/kernels/i8.cpp:132-152) */
int orc_dots_per_row(uint32_t type, int K) {
    return type == ORC_Q6_K ? K / 16 : K / 32;
}

static inline uint16_t rd16(const uint8_t * p) {
    return (uint16_t)(p[0] | (p[1] << 8));
}

/* packed 6-bit (scale, min) pair j of a Q4_K / Q5_K superblock, quant.h:136-144 */
static inline void k4_scale_min(int j, const uint8_t * q, int * sc, int * mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

/* codebook of IQ4_NL / IQ4_XS, quant.h:417 */
static const int8_t kv_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

/* ------------------------------------------------- unpack one 32-value group
 * Integer weight codes of activation group g8 (0..7) of one 256-value
 * superblock, in element order.  Q6_K yields the raw 0..63 codes (the -32 is
 * applied by the caller, as in i8.cpp:152).  */
static void unpack_group(uint32_t type, const uint8_t * sb, int g8, int * q) {
    switch (type) {
    case ORC_Q4_K: { /* i8.cpp:48-58: qs[(g/2)*32+i], low nibble for even g */
        const uint8_t * qs = sb + 16 + (g8 / 2) * 32;
        for (int i = 0; i < 32; i++) {
            q[i] = (g8 & 1) ? (qs[i] >> 4) : (qs[i] & 0xF);
        }
    } break;
    case ORC_Q5_K: { /* i8.cpp:106-114: bit g of qh[i] is the fifth bit */
        const uint8_t * qh = sb + 16;
        const uint8_t * qs = sb + 48 + (g8 / 2) * 32;
        for (int i = 0; i < 32; i++) {
            const int lo = (g8 & 1) ? (qs[i] >> 4) : (qs[i] & 0xF);
            q[i] = lo | (((qh[i] >> g8) & 1) << 4);
        }
    } break;
    case ORC_Q6_K: { /* i8.cpp:132-147; group g8 = scale groups 2*g8 and 2*g8+1 */
        const int blk2 = g8 >> 2, plane = g8 & 3;
        const uint8_t * ql = sb + blk2 * 64 + ((plane & 1) ? 32 : 0);
        const uint8_t * qh = sb + 128 + blk2 * 32;
        for (int i = 0; i < 32; i++) {
            const int lo = (plane >= 2) ? (ql[i] >> 4) : (ql[i] & 0xF);
            q[i] = lo | (((qh[i] >> (2 * plane)) & 3) << 4);
        }
    } break;
    case ORC_IQ4_XS: { /* quant.h:978-991: elements 0..15 low nibbles, 16..31 high */
        const uint8_t * qs = sb + 8 + g8 * 16;
        for (int i = 0; i < 16; i++) {
            q[i] = kv_iq4nl[qs[i] & 0xF];
            q[i + 16] = kv_iq4nl[qs[i] >> 4];
        }
    } break;
    default: { /* Q8_0: 8 blocks of 34 B per 256 values, quant.h:37-41 */
        const int8_t * qs = (const int8_t *)(sb + g8 * B_Q80 + 2);
        for (int i = 0; i < 32; i++) {
            q[i] = qs[i];
        }
    } break;
    }
}

static inline size_t sb_bytes(uint32_t type) {
    return type == ORC_Q8_0 ? 8 * B_Q80 : orc_row_bytes(type, 256);
}

/* ------------------------------------------------------------------ fp32 dequant
 * quant.h:148-232 (Q4_K/Q5_K/Q6_K/Q8_0) and :978-991 (IQ4_XS), same products. */
void orc_dequantize_row(uint32_t type, const void * data, float * y, int64_t n) {
    const uint8_t * p = (const uint8_t *)data;
    const size_t sbb = sb_bytes(type);
    int q[32];
    for (int64_t b = 0; b < n / 256; b++, p += sbb, y += 256) {
        for (int g = 0; g < 8; g++) {
            unpack_group(type, p, g, q);
            if (type == ORC_Q4_K || type == ORC_Q5_K) {
                int sc, mn;
                k4_scale_min(g, p + 4, &sc, &mn);
                const float d1 = orc_h2f(rd16(p)) * (float)sc;
                const float m1 = orc_h2f(rd16(p + 2)) * (float)mn;
                for (int i = 0; i < 32; i++) {
                    y[g * 32 + i] = d1 * (float)q[i] - m1;
                }
            } else if (type == ORC_Q6_K) {
                const float d = orc_h2f(rd16(p + 208));
                const int8_t * sc = (const int8_t *)(p + 192);
                for (int i = 0; i < 32; i++) {
                    y[g * 32 + i] = d * (float)sc[2 * g + i / 16] * (float)(int8_t)(q[i] - 32);
                }
            } else if (type == ORC_IQ4_XS) {
                const uint16_t sh = rd16(p + 2);
                const int ls = ((p[4 + g / 2] >> (4 * (g % 2))) & 0xF) | (((sh >> (2 * g)) & 3) << 4);
                const float dl = orc_h2f(rd16(p)) * (float)(ls - 32);
                for (int i = 0; i < 32; i++) {
                    y[g * 32 + i] = dl * (float)q[i];
                }
            } else {
                const float d = orc_h2f(rd16(p + g * B_Q80));
                for (int i = 0; i < 32; i++) {
                    y[g * 32 + i] = d * (float)q[i];
                }
            }
        }
    }
}

/* ------------------------------------------------------- activation quantizer
 * src/backend/cpu/kernels/xq.cpp:10-50.  Group-major output:
 * x8[(g*TB+t)*32+i], xmeta[2*(g*TB+t)] = f16-truncated max/127 (0 for an all
 * zero group), xsumq[2*(g*TB+t)+{0,1}] = sums of codes 0..15 / 16..31. */
static inline float silu_f(float x) { /* kernels/common.h:31-33 */
    return x / (1.0f + expf(-x));
}

/* RMSNorm of one row, as rmsnorm_row (src/backend/cpu/kernels/common.cpp:685-691): scale =
 * 1 / sqrt(ss / n + eps), out = x * scale * w, with ss = sum of squares in the order of the
 * reference's helper for the host's vector width (common.cpp:259-290, 524-530):
 *   lanes 1   s += a*a, in order (the portable loop; no contraction is assumed)
 *   lanes 8   eight accumulators acc[j] = fma(a, a, acc[j]) over i = 8k + j, then (acc[j] + acc[j+4]),
 *             two horizontal adds: (l0 + l1) + (l2 + l3); a tail of n % 8 elements s += a*a
 *   lanes 16  sixteen accumulators with fma, halved 16 -> 8 -> 4, then (t0 + t2) + (t1 + t3); tail
 *             of n % 16 elements s += a*a */
void orc_rmsnorm(const float * x, const float * w, float * out, int n, float eps, int lanes) {
    float ss = 0.0f;
    int i = 0;
    if (lanes == 8 || lanes == 16) {
        float acc[16] = {0};
        for (; i + lanes <= n; i += lanes) {
            for (int j = 0; j < lanes; j++) {
                acc[j] = fmaf(x[i + j], x[i + j], acc[j]);
            }
        }
        if (lanes == 16) {
            for (int j = 0; j < 8; j++) {
                acc[j] = acc[j + 8] + acc[j];
            }
        }
        for (int j = 0; j < 4; j++) {
            acc[j] = acc[j] + acc[j + 4];
        }
        ss = lanes == 16 ? (acc[0] + acc[2]) + (acc[1] + acc[3]) : (acc[0] + acc[1]) + (acc[2] + acc[3]);
    }
    for (; i < n; i++) {
        ss += x[i] * x[i];
    }
    const float scale = 1.0f / sqrtf(ss / (float)n + eps);
    for (i = 0; i < n; i++) {
        out[i] = x[i] * scale * w[i];
    }
}

void orc_xq(const float * x, const float * up, int x_stride, int up_stride, int8_t * x8, float * xmeta,
            int32_t * xsumq, int TB, int K) {
    const int G = K / 32;
    for (int gid = 0; gid < TB * G; gid++) {
        const int t = gid / G, g = gid % G;
        float v[32], mx = 0.0f;
        for (int i = 0; i < 32; i++) {
            float a = x[(size_t)t * x_stride + g * 32 + i];
            if (up) {
                a = silu_f(a) * up[(size_t)t * up_stride + g * 32 + i];
            }
            v[i] = a;
            const float aa = fabsf(a);
            mx = mx < aa ? aa : mx;
        }
        const float inv = mx > 0.0f ? 127.0f / mx : 0.0f;
        const size_t gi = (size_t)g * TB + t;
        int32_t s[2] = {0, 0};
        for (int i = 0; i < 32; i++) {
            float r = roundf(v[i] * inv);
            r = r > 127.0f ? 127.0f : r;
            r = r < -127.0f ? -127.0f : r;
            x8[gi * 32 + i] = (int8_t)(int32_t)r;
            s[i >> 4] += (int32_t)r;
        }
        xmeta[gi * 2] = orc_h2f(orc_f2h(mx > 0.0f ? mx / 127.0f : 0.0f));
        xmeta[gi * 2 + 1] = 0.0f;
        xsumq[gi * 2] = s[0];
        xsumq[gi * 2 + 1] = s[1];
    }
}

/* ---------------------------------------------------- int32 per-group dots
 * The exact integer sums the reference forms inside q4k/q5k/q6k_i8_block
 * (i8.cpp:57, :117, :149) but never exposes.  wd[row*D + j]: j = 32-value group
 * index, or for Q6_K the 16-value scale group (raw codes 0..63, no -32). */
void orc_block_dots(uint32_t type, const void * w, int K, int n_rows, const int8_t * x8, int TB, int t,
                    int32_t * wd) {
    const int nb = K / 256, D = orc_dots_per_row(type, K);
    const size_t sbb = sb_bytes(type);
    for (int r = 0; r < n_rows; r++) {
        int q[32];
        const uint8_t * row = (const uint8_t *)w + (size_t)r * nb * sbb;
        for (int b = 0; b < nb; b++) {
            for (int g = 0; g < 8; g++) {
                const int8_t * xv = x8 + ((size_t)(b * 8 + g) * TB + t) * 32;
                unpack_group(type, row + b * sbb, g, q);
                int32_t a0 = 0, a1 = 0;
                for (int i = 0; i < 16; i++) {
                    a0 += q[i] * xv[i];
                    a1 += q[i + 16] * xv[i + 16];
                }
                if (type == ORC_Q6_K) {
                    wd[(size_t)r * D + (b * 8 + g) * 2] = a0;
                    wd[(size_t)r * D + (b * 8 + g) * 2 + 1] = a1;
                } else {
                    wd[(size_t)r * D + b * 8 + g] = a0 + a1;
                }
            }
        }
    }
}

/* ------------------------------------------------------------ one output value
 * Per-group term of token t, in the reference's fp32 association:
 *   Q4_K/Q5_K  xm * ((d*sc)*(float)wd - (dmin*m)*(float)(s0+s1))   i8.cpp:59, :119, :236, :283
 *   Q6_K       (xm * (d*(float)sc_s)) * (float)(wd - 32*xs_half)     i8.cpp:150-152, :308-312
 *   Q8_0       (xm * d) * (float)wd                                  q4exp.cpp:456-458
 *   IQ4_XS     (xm * (d*(float)(ls-32))) * (float)wd     no reference integer kernel: dequant
 *              formula of quant.h:978-991 applied in the Q6_K association
 * `flat` selects the accumulation order: 0 = per-superblock partial sums added
 * in block order (i8_row, i8.cpp:157-190), 1 = one running sum over all groups
 * (the tiled GEMM, i8.cpp:316-349, and q8_0_down_row). */
static float row_value(uint32_t type, const uint8_t * row, const int8_t * x8, const float * xmeta,
                       const int32_t * xsumq, int TB, int t, int K, int flat, double * abs_sum) {
    const int nb = K / 256;
    const size_t sbb = sb_bytes(type);
    int q[32];
    float total = 0.0f;
    double ab = 0.0;
    for (int b = 0; b < nb; b++) {
        const uint8_t * sb = row + b * sbb;
        float acc = flat ? total : 0.0f;
        for (int g = 0; g < 8; g++) {
            const size_t ai = (size_t)(b * 8 + g) * TB + t;
            const int8_t * xv = x8 + ai * 32;
            const float xm = xmeta[ai * 2];
            unpack_group(type, sb, g, q);
            int32_t a0 = 0, a1 = 0;
            for (int i = 0; i < 16; i++) {
                a0 += q[i] * xv[i];
                a1 += q[i + 16] * xv[i + 16];
            }
            if (type == ORC_Q4_K || type == ORC_Q5_K) {
                int sc, mn;
                k4_scale_min(g, sb + 4, &sc, &mn);
                const float dsc = orc_h2f(rd16(sb)) * (float)sc;
                const float dmm = orc_h2f(rd16(sb + 2)) * (float)mn;
                const float p1 = dsc * (float)(a0 + a1);
                const float p2 = dmm * (float)(xsumq[ai * 2] + xsumq[ai * 2 + 1]);
                acc += xm * (p1 - p2);
                ab += fabs((double)xm * p1) + fabs((double)xm * p2);
            } else if (type == ORC_Q6_K) {
                const float d = orc_h2f(rd16(sb + 208));
                const int8_t * sc = (const int8_t *)(sb + 192);
                const float ds0 = d * (float)sc[2 * g], ds1 = d * (float)sc[2 * g + 1];
                const float t0 = xm * ds0 * (float)(a0 - 32 * xsumq[ai * 2]);
                acc += t0;
                const float t1 = xm * ds1 * (float)(a1 - 32 * xsumq[ai * 2 + 1]);
                acc += t1;
                ab += fabs((double)xm * ds0 * a0) + fabs((double)xm * ds0 * 32.0 * xsumq[ai * 2]);
                ab += fabs((double)xm * ds1 * a1) + fabs((double)xm * ds1 * 32.0 * xsumq[ai * 2 + 1]);
            } else if (type == ORC_IQ4_XS) {
                const uint16_t sh = rd16(sb + 2);
                const int ls = ((sb[4 + g / 2] >> (4 * (g % 2))) & 0xF) | (((sh >> (2 * g)) & 3) << 4);
                const float dl = orc_h2f(rd16(sb)) * (float)(ls - 32);
                const float tt = xm * dl * (float)(a0 + a1);
                acc += tt;
                ab += fabs((double)tt);
            } else {
                const float d = orc_h2f(rd16(sb + g * B_Q80));
                const float tt = xm * d * (float)(a0 + a1);
                acc += tt;
                ab += fabs((double)tt);
            }
        }
        total = flat ? acc : total + acc;
    }
    if (abs_sum) {
        *abs_sum = ab;
    }
    return total;
}

static inline int type_is_flat(uint32_t type) {
    return type == ORC_Q8_0; /* q8_0_down_row keeps one running sum, q4exp.cpp:446-459 */
}

float orc_row(uint32_t type, const void * wrow, const int8_t * x8, const float * xmeta, const int32_t * xsumq,
              int TB, int t, int K) {
    return row_value(type, (const uint8_t *)wrow, x8, xmeta, xsumq, TB, t, K, type_is_flat(type), NULL);
}

/* sum of |terms| of the same row: the yardstick the fp32 tolerance is scaled by */
double orc_row_abs(uint32_t type, const void * wrow, const int8_t * x8, const float * xmeta, const int32_t * xsumq,
                   int TB, int t, int K) {
    double ab = 0.0;
    (void)row_value(type, (const uint8_t *)wrow, x8, xmeta, xsumq, TB, t, K, 0, &ab);
    return ab;
}

/* ------------------------------------------------------------- GEMV / GEMM
 * cpu_i8_gemv (i8.cpp:498-516) for TB == 1: out[row] = alpha*row (+ residual[row]).
 * cpu_i8_gemm (i8.cpp:518-546): TB >= 2 takes the tiled form whose running sum
 * is flat over groups (i8.cpp:316-349) and whose epilogue is
 * val = alpha*acc; val += residual[t*out_stride+row] (i8.cpp:364-373). */
typedef struct {
    const orc_seg * s;
    int TB, flat;
    size_t rb;
    double * abs_out;
} gemm_ctx;

static void gemm_row(int row, void * p) {
    const gemm_ctx * c = (const gemm_ctx *)p;
    const orc_seg * s = c->s;
    const uint8_t * wr = (const uint8_t *)s->w + (size_t)row * c->rb;
    for (int t = 0; t < c->TB; t++) {
        double ab = 0.0;
        float v = s->alpha * row_value(s->type, wr, s->x8, s->xmeta, s->xsumq, c->TB, t, s->K, c->flat, &ab);
        const size_t o = (size_t)t * s->out_stride + row;
        if (s->residual) {
            v += s->residual[o];
        }
        if (s->out) {
            s->out[o] = v;
        }
        if (c->abs_out) {
            c->abs_out[o] = ab * fabs((double)s->alpha);
        }
    }
}

static void gemm_impl(const orc_seg * s, int TB, double * abs_out) {
    gemm_ctx c = {s, TB, (TB >= 2) || type_is_flat(s->type), orc_row_bytes(s->type, s->K), abs_out};
    par_for(s->n_rows, gemm_row, &c);
}

void orc_i8_gemm(const orc_seg * seg, int TB) {
    gemm_impl(seg, TB, NULL);
}

void orc_i8_gemm_abs(const orc_seg * seg, int TB, double * abs_out) {
    orc_seg s = *seg;
    s.out = NULL;
    gemm_impl(&s, TB, abs_out);
}

/* ------------------------------------------------------------------- MoE router
 * src/backend/cpu/kernels/moe.cpp:72-137.  F32 router weights, double logits
 * accumulation (the non-fast branch), softmax over ALL experts with a
 * sequential fp32 sum, top-k by rank counting (ties to the lower index),
 * weights divided by max(sum of the selected, 6.103515625e-5). */
void orc_moe_route_logits(int n_tok, int n_expert, int top_k, float * logits, int32_t * ids, float * wts) {
    for (int t = 0; t < n_tok; t++) {
        float * p = logits + (size_t)t * n_expert;
        float mx = -3.402823466e38f;
        for (int e = 0; e < n_expert; e++) {
            mx = fmaxf(mx, p[e]);
        }
        float sum = 0.f;
        for (int e = 0; e < n_expert; e++) {
            p[e] = expf(p[e] - mx);
            sum += p[e];
        }
        const float inv = 1.f / sum;
        for (int e = 0; e < n_expert; e++) {
            p[e] *= inv;
        }
        float wsum = 0.f;
        for (int e = 0; e < n_expert; e++) {
            int rank = 0;
            for (int f = 0; f < n_expert; f++) {
                rank += (p[f] > p[e]) || (p[f] == p[e] && f < e);
            }
            if (rank < top_k) {
                ids[(size_t)t * top_k + rank] = e;
                wts[(size_t)t * top_k + rank] = p[e];
                wsum += p[e];
            }
        }
        const float den = fmaxf(wsum, 6.103515625e-5f);
        for (int j = 0; j < top_k; j++) {
            wts[(size_t)t * top_k + j] /= den;
        }
    }
}

void orc_moe_route(const float * x, int x_stride, const float * gate_inp, int n_tok, int n_embd, int n_expert,
                   int top_k, float * logits, int32_t * ids, float * wts) {
    for (int t = 0; t < n_tok; t++) {
        for (int e = 0; e < n_expert; e++) {
            double a = 0;
            for (int k = 0; k < n_embd; k++) {
                a += (double)gate_inp[(size_t)e * n_embd + k] * (double)x[(size_t)t * x_stride + k];
            }
            logits[(size_t)t * n_expert + e] = (float)a;
        }
    }
    orc_moe_route_logits(n_tok, n_expert, top_k, logits, ids, wts);
}

/* ------------------------------------------------------- routed experts, int8
 * src/backend/cpu/kernels/moe.cpp:476-559 (cpu_moe_experts_i8): the token row is
 * quantized once (quant_row_1, :450-471 = the cpu_xq rule with TB = 1), each
 * pair runs gate and up from the GGUF blocks (cpu_i8_gemv1_chunked), forms
 * h = silu(g)*u in fp32, re-quantizes h per 32-group and runs down.  The
 * reference's down branch handles Q5_1/Q8_0/its int8 store; a K-quant down
 * plane is the same cpu_i8_gemv1_chunked on the plane pointer.
 * acc[pair*acc_stride + r] is the UNWEIGHTED expert output; h_out (optional)
 * receives the [pairs][n_ff] intermediate. */
typedef struct {
    const void *gate, *up, *down;
    uint32_t gt, ut, dt;
    size_t gp, upl, dp;
    int n_embd, n_ff, x_stride, top_k, acc_stride;
    const float * x;
    const int32_t * ids;
    float *h_out, *acc;
} moe_ctx;

static void moe_pair(int pr, void * p) {
    const moe_ctx * c = (const moe_ctx *)p;
    const int n_embd = c->n_embd, n_ff = c->n_ff;
    const int G = n_embd / 32, Gd = n_ff / 32;
    const size_t grb = orc_row_bytes(c->gt, n_embd), urb = orc_row_bytes(c->ut, n_embd);
    const size_t drb = orc_row_bytes(c->dt, n_ff);
    const int t = pr / c->top_k, e = c->ids[pr];
    int8_t * x8 = (int8_t *)malloc((size_t)n_embd + n_ff);
    int8_t * h8 = x8 + n_embd;
    float * xm = (float *)malloc(sizeof(float) * 2 * (size_t)(G + Gd));
    float * hm = xm + 2 * G;
    int32_t * xs = (int32_t *)malloc(sizeof(int32_t) * 2 * (size_t)(G + Gd));
    int32_t * hs = xs + 2 * G;
    float * h = (float *)malloc(sizeof(float) * (size_t)n_ff);
    orc_xq(c->x + (size_t)t * c->x_stride, NULL, n_embd, 0, x8, xm, xs, 1, n_embd);
    const uint8_t * gp = (const uint8_t *)c->gate + (size_t)e * c->gp;
    const uint8_t * upp = (const uint8_t *)c->up + (size_t)e * c->upl;
    const uint8_t * dp = (const uint8_t *)c->down + (size_t)e * c->dp;
    for (int i = 0; i < n_ff; i++) {
        const float gv = orc_row(c->gt, gp + (size_t)i * grb, x8, xm, xs, 1, 0, n_embd);
        const float uv = orc_row(c->ut, upp + (size_t)i * urb, x8, xm, xs, 1, 0, n_embd);
        h[i] = silu_f(gv) * uv;
        if (c->h_out) {
            c->h_out[(size_t)pr * n_ff + i] = h[i];
        }
    }
    orc_xq(h, NULL, n_ff, 0, h8, hm, hs, 1, n_ff);
    for (int r = 0; r < n_embd; r++) {
        c->acc[(size_t)pr * c->acc_stride + r] = orc_row(c->dt, dp + (size_t)r * drb, h8, hm, hs, 1, 0, n_ff);
    }
    free(x8);
    free(xm);
    free(xs);
    free(h);
}

void orc_moe_experts_i8(const void * gate, const void * up, const void * down, uint32_t gate_type, uint32_t up_type,
                        uint32_t down_type, size_t gate_plane, size_t up_plane, size_t down_plane, int n_embd,
                        int n_ff, const float * x, int x_stride, int n_tok, int top_k, const int32_t * ids,
                        float * h_out, float * acc, int acc_stride) {
    moe_ctx c = {gate, up, down, gate_type, up_type, down_type, gate_plane, up_plane, down_plane,
                 n_embd, n_ff, x_stride, top_k, acc_stride, x, ids, h_out, acc};
    par_for(n_tok * top_k, moe_pair, &c);
}

/* src/backend/cpu/kernels/moe.cpp:562-574: out[t] += (float) sum_j (double)w*acc */
void orc_moe_reduce(const float * acc, const float * wts, int top_k, int n_tok, int n_embd, int acc_stride,
                    float * out, int out_stride) {
    for (int t = 0; t < n_tok; t++) {
        for (int e = 0; e < n_embd; e++) {
            double a = 0;
            for (int j = 0; j < top_k; j++) {
                const size_t pr = (size_t)t * top_k + j;
                a += (double)wts[pr] * acc[pr * (size_t)acc_stride + e];
            }
            out[(size_t)t * out_stride + e] += (float)a;
        }
    }
}
