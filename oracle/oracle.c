/* TEST INFRASTRUCTURE ONLY -- see oracle.h.  Plain-C CPU restatement of the
 * reference's hot-path algorithms.  Built with -ffp-contract=off and without
 * fast-math so every float32 sum is the same sequence of IEEE operations the
 * reference's CPU code performs (one accumulator, k ascending). */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>

/* ------------------------------------------------------------------ threads */

static int g_threads = 0;

int orc_num_threads(void) {
    if (g_threads <= 0) {
        const char* e = getenv("ORC_THREADS");
        g_threads = e ? atoi(e) : 8;
        if (g_threads <= 0) g_threads = 1;
        if (g_threads > 256) g_threads = 256;
    }
    return g_threads;
}
void orc_set_num_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }

typedef void (*range_fn)(int64_t lo, int64_t hi, void* arg);
typedef struct { range_fn fn; void* arg; int64_t lo, hi; } RangeJob;
static void* range_tramp(void* p) { RangeJob* j = (RangeJob*)p; j->fn(j->lo, j->hi, j->arg); return 0; }

/* Splits [0,n) into contiguous slices, one per thread.  Every output element is
 * produced by exactly one thread with a fixed operation order, so results do
 * not depend on the thread count. */
static void parallel_for(int64_t n, range_fn fn, void* arg) {
    int T = orc_num_threads();
    if (T > n) T = (int)(n > 0 ? n : 1);
    if (T <= 1) { fn(0, n, arg); return; }
    pthread_t th[256]; RangeJob jobs[256];
    for (int t = 0; t < T; t++) {
        jobs[t].fn = fn; jobs[t].arg = arg;
        jobs[t].lo = n * t / T; jobs[t].hi = n * (t + 1) / T;
        pthread_create(&th[t], 0, range_tramp, &jobs[t]);
    }
    for (int t = 0; t < T; t++) pthread_join(th[t], 0);
}

/* ----------------------------------------------------------------- rounding */

typedef union { float f; uint32_t u; } F32Bits;

float orc_bf16_round(float f) {
    F32Bits b; b.f = f;
    b.u += 0x7FFFu + ((b.u >> 16) & 1u);
    b.u &= 0xFFFF0000u;
    return b.f;
}

float orc_tf32_trunc(float f) {
    F32Bits b; b.f = f;
    b.u &= 0xFFFFE000u;
    return b.f;
}

void orc_round_array(const float* in, float* out, int64_t n, int mode) {
    if (mode == ORC_BF16) for (int64_t i = 0; i < n; i++) out[i] = orc_bf16_round(in[i]);
    else if (mode == ORC_TF32) for (int64_t i = 0; i < n; i++) out[i] = orc_tf32_trunc(in[i]);
    else if (in != out) memcpy(out, in, (size_t)n * sizeof(float));
}

static float rnd(float v, int mode) {
    return mode == ORC_BF16 ? orc_bf16_round(v) : mode == ORC_TF32 ? orc_tf32_trunc(v) : v;
}

/* --------------------------------------------------------------------- GEMM */

typedef struct {
    const float* a; const float* b; float* c;   /* packed op(A) [M,K], op(B) [K,N]; C with ldc */
    int M, N, K, ldc; float alpha, beta;
} GemmJob;

/* rows [lo,hi): acc[j] walks k = 0..K-1 for every j, i.e. each output element is
 * ((0 + a0*b0) + a1*b1) + ... exactly like the i-j-k loop of tensor_matmul2d. */
static void gemm_rows(int64_t lo, int64_t hi, void* arg) {
    GemmJob* g = (GemmJob*)arg;
    int N = g->N, K = g->K;
    float* acc = (float*)malloc((size_t)N * sizeof(float));
    for (int64_t i = lo; i < hi; i++) {
        for (int j = 0; j < N; j++) acc[j] = 0.0f;
        const float* ai = g->a + i * K;
        for (int k = 0; k < K; k++) {
            float av = ai[k];
            const float* bk = g->b + (int64_t)k * N;
            for (int j = 0; j < N; j++) acc[j] += av * bk[j];
        }
        float* ci = g->c + i * g->ldc;
        if (g->beta == 0.0f) {
            if (g->alpha == 1.0f) for (int j = 0; j < N; j++) ci[j] = acc[j];
            else for (int j = 0; j < N; j++) ci[j] = g->alpha * acc[j];
        } else {
            for (int j = 0; j < N; j++) ci[j] = g->alpha * acc[j] + g->beta * ci[j];
        }
    }
    free(acc);
}

static float* pack_op(const float* X, int rows, int cols, int ld, int trans, int mode) {
    /* returns op(X) as contiguous [rows, cols]; trans: X stored [cols, rows] */
    float* p = (float*)malloc((size_t)rows * cols * sizeof(float) + 16);
    if (!trans) {
        for (int i = 0; i < rows; i++)
            for (int j = 0; j < cols; j++) p[(int64_t)i * cols + j] = rnd(X[(int64_t)i * ld + j], mode);
    } else {
        for (int j = 0; j < cols; j++)
            for (int i = 0; i < rows; i++) p[(int64_t)i * cols + j] = rnd(X[(int64_t)j * ld + i], mode);
    }
    return p;
}

void orc_gemm(int ta, int tb, const float* A, const float* B, float* C,
              int M, int N, int K, int lda, int ldb, int ldc,
              int batch, int64_t sA, int64_t sB, int64_t sC,
              float alpha, float beta, int mode) {
    for (int z = 0; z < batch; z++) {
        float* pa = pack_op(A + z * sA, M, K, lda, ta, mode);
        float* pb = pack_op(B + z * sB, K, N, ldb, tb, mode);
        GemmJob g = { pa, pb, C + z * sC, M, N, K, ldc, alpha, beta };
        parallel_for(M, gemm_rows, &g);
        free(pa); free(pb);
    }
}

void orc_gemm_f64(int ta, int tb, const float* A, const float* B, double* C,
                  int M, int N, int K, int lda, int ldb, int ldc) {
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            double s = 0.0;
            for (int k = 0; k < K; k++) {
                double a = ta ? A[(int64_t)k * lda + i] : A[(int64_t)i * lda + k];
                double b = tb ? B[(int64_t)j * ldb + k] : B[(int64_t)k * ldb + j];
                s += a * b;
            }
            C[(int64_t)i * ldc + j] = s;
        }
}

void orc_gemm_bias(const float* A, const float* B, const float* bias, const float* residual,
                   float* C, int M, int N, int K, int mode) {
    orc_gemm(0, 0, A, B, C, M, N, K, K, N, N, 1, 0, 0, 0, 1.0f, 0.0f, mode);
    for (int64_t i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            float v = C[i * N + j] + (bias ? bias[j] : 0.0f);
            if (residual) v += residual[i * N + j];
            C[i * N + j] = v;
        }
}

void orc_colsum_acc(const float* in, float* out, int rows, int cols) {
    /* the reference sums 8 strided partials then the 8 partials in order */
    for (int c = 0; c < cols; c++) {
        float part[8];
        for (int ty = 0; ty < 8; ty++) {
            float s = 0.0f;
            for (int r = ty; r < rows; r += 8) s += in[(int64_t)r * cols + c];
            part[ty] = s;
        }
        float t = part[0];
        for (int k = 1; k < 8; k++) t += part[k];
        out[c] += t;
    }
}

/* ------------------------------------------------------------------ RMSNorm */

void orc_rmsnorm_fwd(const float* x, const float* w, float* out, float* rinv, int rows, int cols, float eps) {
    for (int64_t n = 0; n < rows; n++) {
        const float* xr = x + n * cols;
        float ss = 0.0f;
        for (int i = 0; i < cols; i++) ss += xr[i] * xr[i];
        float ms = ss / (float)cols;
        float r = 1.0f / (float)sqrt((double)(ms + eps));
        if (rinv) rinv[n] = r;
        for (int i = 0; i < cols; i++) out[n * cols + i] = xr[i] * r * w[i];
    }
}

void orc_rmsnorm_bwd(const float* x, const float* w, const float* rinv, const float* dy,
                     float* dx, float* dw, int rows, int cols) {
    float* wt = (float*)malloc((size_t)rows * cols * sizeof(float));
    for (int64_t n = 0; n < rows; n++) {
        const float* xr = x + n * cols; const float* dyr = dy + n * cols;
        float r = rinv[n], r3 = r * r * r, S = 0.0f;
        for (int i = 0; i < cols; i++) S += dyr[i] * w[i] * xr[i];
        for (int j = 0; j < cols; j++) {
            dx[n * cols + j] += w[j] * r * dyr[j] - (r3 / (float)cols) * xr[j] * S;
            wt[n * cols + j] = dyr[j] * xr[j] * r;
        }
    }
    orc_colsum_acc(wt, dw, rows, cols);
    free(wt);
}

/* --------------------------------------------------------------------- RoPE */

void orc_rope_tables(int T, int hd, float base, float* cos_t, float* sin_t) {
    int half = hd / 2;
    for (int pos = 0; pos < T; pos++)
        for (int k = 0; k < half; k++) {
            float exponent = -(2.0f * (float)k) / (float)hd;
            float theta = powf(base, exponent);
            float angle = (float)pos * theta;
            cos_t[pos * half + k] = cosf(angle);
            sin_t[pos * half + k] = sinf(angle);
        }
}

void orc_qkv_rope_split(const float* qkv, const float* cos_t, const float* sin_t,
                        float* Q, float* K, float* V, int B, int T, int H, int hd) {
    int half = hd / 2, D = H * hd;
    for (int64_t n = 0; n < (int64_t)B * T; n++) {
        int t = (int)(n % T); int64_t b = n / T;
        const float* row = qkv + n * 3 * D;
        for (int h = 0; h < H; h++)
            for (int k = 0; k < half; k++) {
                int c0 = h * hd + 2 * k;
                float c = cos_t[t * half + k], s = sin_t[t * half + k];
                int64_t o = ((b * H + h) * T + t) * hd + 2 * k;
                float q0 = row[c0], q1 = row[c0 + 1];
                Q[o] = q0 * c - q1 * s; Q[o + 1] = q0 * s + q1 * c;
                float k0 = row[D + c0], k1 = row[D + c0 + 1];
                K[o] = k0 * c - k1 * s; K[o + 1] = k0 * s + k1 * c;
                V[o] = row[2 * D + c0]; V[o + 1] = row[2 * D + c0 + 1];
            }
    }
}

void orc_qkv_rope_merge_bwd(const float* dQ, const float* dK, const float* dV,
                            const float* cos_t, const float* sin_t, float* dqkv,
                            int B, int T, int H, int hd) {
    int half = hd / 2, D = H * hd;
    for (int64_t n = 0; n < (int64_t)B * T; n++) {
        int t = (int)(n % T); int64_t b = n / T;
        float* row = dqkv + n * 3 * D;
        for (int h = 0; h < H; h++)
            for (int k = 0; k < half; k++) {
                int c0 = h * hd + 2 * k;
                float c = cos_t[t * half + k], s = sin_t[t * half + k];
                int64_t o = ((b * H + h) * T + t) * hd + 2 * k;
                float a0 = dQ[o], a1 = dQ[o + 1];
                row[c0] = a0 * c + a1 * s; row[c0 + 1] = -a0 * s + a1 * c;
                float b0 = dK[o], b1 = dK[o + 1];
                row[D + c0] = b0 * c + b1 * s; row[D + c0 + 1] = -b0 * s + b1 * c;
                row[2 * D + c0] = dV[o]; row[2 * D + c0 + 1] = dV[o + 1];
            }
    }
}

/* ---------------------------------------------------------------- attention */

typedef struct {
    const float *Q, *K, *V, *dO; float *O, *P, *dQ, *dK, *dV;
    int T, hd; float scale; int mode;
} AttnJob;

/* one (batch, head): S = Q K^T; S*scale + mask; softmax rows; O = P V */
static void attn_fwd_heads(int64_t lo, int64_t hi, void* arg) {
    AttnJob* a = (AttnJob*)arg;
    int T = a->T, hd = a->hd, mode = a->mode;
    float* p = (float*)malloc((size_t)T * sizeof(float));
    for (int64_t z = lo; z < hi; z++) {
        const float* Q = a->Q + z * T * hd; const float* K = a->K + z * T * hd; const float* V = a->V + z * T * hd;
        float* O = a->O + z * T * hd;
        for (int i = 0; i < T; i++) {
            float mx = -3.0e38f;
            for (int j = 0; j < T; j++) {
                float s = 0.0f;
                for (int k = 0; k < hd; k++) s += rnd(Q[i * hd + k], mode) * rnd(K[j * hd + k], mode);
                float v = s * a->scale + ((j <= i) ? 0.0f : -1e9f);
                p[j] = v;
                if (v > mx) mx = v;
            }
            float sum = 0.0f;
            for (int j = 0; j < T; j++) { float e = expf(p[j] - mx); p[j] = e; sum += e; }
            for (int j = 0; j < T; j++) p[j] /= sum;
            if (a->P) memcpy(a->P + (z * T + i) * T, p, (size_t)T * sizeof(float));
            for (int d = 0; d < hd; d++) {
                float s = 0.0f;
                for (int j = 0; j < T; j++) s += rnd(p[j], mode) * rnd(V[j * hd + d], mode);
                O[i * hd + d] = s;
            }
        }
    }
    free(p);
}

void orc_attention_fwd(const float* Q, const float* K, const float* V, float* O, float* P_out,
                       int BH, int T, int hd, float scale, int mode) {
    AttnJob a; memset(&a, 0, sizeof(a));
    a.Q = Q; a.K = K; a.V = V; a.O = O; a.P = P_out; a.T = T; a.hd = hd; a.scale = scale; a.mode = mode;
    parallel_for(BH, attn_fwd_heads, &a);
}

/* backward as the reference GPU trainer sequences it (model/gpu_train.c:435-455):
 * dV = P^T dO; dP = dO V^T; dS = P*(dP - <dP,P>)*scale; dQ = dS K; dK = dS^T Q */
static void attn_bwd_heads(int64_t lo, int64_t hi, void* arg) {
    AttnJob* a = (AttnJob*)arg;
    int T = a->T, hd = a->hd, mode = a->mode;
    float* P = (float*)malloc((size_t)T * T * sizeof(float));
    float* dS = (float*)malloc((size_t)T * T * sizeof(float));
    for (int64_t z = lo; z < hi; z++) {
        const float* Q = a->Q + z * T * hd; const float* K = a->K + z * T * hd;
        const float* V = a->V + z * T * hd; const float* dO = a->dO + z * T * hd;
        float* dQ = a->dQ + z * T * hd; float* dK = a->dK + z * T * hd; float* dV = a->dV + z * T * hd;
        for (int i = 0; i < T; i++) {
            float* p = P + (int64_t)i * T;
            float mx = -3.0e38f;
            for (int j = 0; j < T; j++) {
                float s = 0.0f;
                for (int k = 0; k < hd; k++) s += rnd(Q[i * hd + k], mode) * rnd(K[j * hd + k], mode);
                float v = s * a->scale + ((j <= i) ? 0.0f : -1e9f);
                p[j] = v; if (v > mx) mx = v;
            }
            float sum = 0.0f;
            for (int j = 0; j < T; j++) { float e = expf(p[j] - mx); p[j] = e; sum += e; }
            for (int j = 0; j < T; j++) p[j] /= sum;
        }
        for (int j = 0; j < T; j++)
            for (int d = 0; d < hd; d++) {
                float s = 0.0f;
                for (int i = 0; i < T; i++) s += rnd(P[(int64_t)i * T + j], mode) * rnd(dO[i * hd + d], mode);
                dV[j * hd + d] = s;
            }
        for (int i = 0; i < T; i++) {
            float* ds = dS + (int64_t)i * T; const float* p = P + (int64_t)i * T;
            float dot = 0.0f;
            for (int j = 0; j < T; j++) {
                float s = 0.0f;
                for (int d = 0; d < hd; d++) s += rnd(dO[i * hd + d], mode) * rnd(V[j * hd + d], mode);
                ds[j] = s; dot += s * p[j];
            }
            for (int j = 0; j < T; j++) ds[j] = p[j] * (ds[j] - dot) * a->scale;
        }
        for (int i = 0; i < T; i++)
            for (int d = 0; d < hd; d++) {
                float s = 0.0f;
                for (int j = 0; j < T; j++) s += rnd(dS[(int64_t)i * T + j], mode) * rnd(K[j * hd + d], mode);
                dQ[i * hd + d] = s;
            }
        for (int j = 0; j < T; j++)
            for (int d = 0; d < hd; d++) {
                float s = 0.0f;
                for (int i = 0; i < T; i++) s += rnd(dS[(int64_t)i * T + j], mode) * rnd(Q[i * hd + d], mode);
                dK[j * hd + d] = s;
            }
    }
    free(P); free(dS);
}

void orc_attention_bwd(const float* Q, const float* K, const float* V, const float* dO,
                       float* dQ, float* dK, float* dV,
                       int BH, int T, int hd, float scale, int mode) {
    AttnJob a; memset(&a, 0, sizeof(a));
    a.Q = Q; a.K = K; a.V = V; a.dO = dO; a.dQ = dQ; a.dK = dK; a.dV = dV;
    a.T = T; a.hd = hd; a.scale = scale; a.mode = mode;
    parallel_for(BH, attn_bwd_heads, &a);
}

void orc_heads_merge(const float* O, float* out, int B, int T, int H, int hd) {
    for (int64_t b = 0; b < B; b++) for (int h = 0; h < H; h++) for (int t = 0; t < T; t++) for (int d = 0; d < hd; d++)
        out[(b * T + t) * (int64_t)(H * hd) + h * hd + d] = O[((b * H + h) * T + t) * hd + d];
}

void orc_heads_split(const float* dout, float* dO, int B, int T, int H, int hd) {
    for (int64_t b = 0; b < B; b++) for (int h = 0; h < H; h++) for (int t = 0; t < T; t++) for (int d = 0; d < hd; d++)
        dO[((b * H + h) * T + t) * hd + d] = dout[(b * T + t) * (int64_t)(H * hd) + h * hd + d];
}

/* ------------------------------------------------- SwiGLU, embedding, loss */

void orc_swiglu_fwd(const float* gu, float* h, int rows, int F) {
    for (int64_t n = 0; n < rows; n++)
        for (int j = 0; j < F; j++) {
            float g = gu[n * 2 * F + j], u = gu[n * 2 * F + F + j];
            float sg = 1.0f / (1.0f + expf(-g));
            h[n * F + j] = g * sg * u;
        }
}

void orc_swiglu_bwd(const float* gu, const float* dh, float* dgu, int rows, int F) {
    for (int64_t n = 0; n < rows; n++)
        for (int j = 0; j < F; j++) {
            float g = gu[n * 2 * F + j], u = gu[n * 2 * F + F + j];
            float sg = 1.0f / (1.0f + expf(-g));
            float d = dh[n * F + j];
            float dsilu = d * u;
            dgu[n * 2 * F + j] = dsilu * sg + dsilu * g * sg * (1.0f - sg);
            dgu[n * 2 * F + F + j] = d * g * sg;
        }
}

void orc_embed_fwd(const float* E, const uint32_t* ids, float* x, int rows, int D) {
    for (int64_t n = 0; n < rows; n++) memcpy(x + n * D, E + (int64_t)ids[n] * D, (size_t)D * sizeof(float));
}

void orc_embed_bwd(const float* dx, const uint32_t* ids, float* dE, int rows, int D) {
    /* rows visited in ascending order for every column: fixed summation order */
    for (int64_t n = 0; n < rows; n++)
        for (int j = 0; j < D; j++) dE[(int64_t)ids[n] * D + j] += dx[n * D + j];
}

typedef struct { float* logits; const uint32_t* targets; float* loss_rows; int V, ld; float gs; } CEJob;

static void ce_rows(int64_t lo, int64_t hi, void* arg) {
    CEJob* c = (CEJob*)arg;
    for (int64_t n = lo; n < hi; n++) {
        float* z = c->logits + n * c->ld;
        uint32_t t = c->targets[n];
        float mx = z[0];
        for (int j = 1; j < c->V; j++) if (z[j] > mx) mx = z[j];
        float sum = 0.0f;
        for (int j = 0; j < c->V; j++) sum += expf(z[j] - mx);
        c->loss_rows[n] = (float)log((double)sum) + mx - z[t];
        float inv = 1.0f / sum;
        for (int j = 0; j < c->V; j++) {
            float p = expf(z[j] - mx) * inv;
            if (j == (int)t) p -= 1.0f;
            z[j] = p * c->gs;
        }
    }
}

void orc_cross_entropy(float* logits, const uint32_t* targets, float* loss_rows,
                       int rows, int V, int ld, float grad_scale) {
    CEJob c = { logits, targets, loss_rows, V, ld, grad_scale };
    parallel_for(rows, ce_rows, &c);
}

/* --------------------------------------------------------------------- Adam */

void orc_adam(float* p, const float* g, float* m, float* v, int64_t n,
              float lr, float b1, float b2, float eps, float bc1, float bc2, float grad_scale) {
    for (int64_t i = 0; i < n; i++) {
        float gi = g[i] * grad_scale;
        float mi = b1 * m[i] + (1.0f - b1) * gi;
        float vi = b2 * v[i] + (1.0f - b2) * gi * gi;
        m[i] = mi; v[i] = vi;
        float m_hat = mi / bc1, v_hat = vi / bc2;
        p[i] -= lr * m_hat / (sqrtf(v_hat) + eps);
    }
}

double orc_grad_norm(const float* g, int64_t n) {
    double ss = 0.0;
    for (int64_t i = 0; i < n; i++) ss += (double)g[i] * (double)g[i];
    return sqrt(ss);
}

/* -------------------------------------------------------------- whole model */

/* flat parameter layout, lm_collect_params order (model/lm_model.c:84-98;
 * model/gpu_train.c:8-13): embed [V,D]; per layer attn_norm [D], w_qkv [D,3D],
 * b_qkv [3D], wo [D,D], bo [D], ffn_norm [D], w_gu [D,2F], b_gu [2F],
 * w_down [F,D], b_down [D]; final_norm [D]. */
enum { PK_ATTN_NORM = 0, PK_WQKV, PK_BQKV, PK_WO, PK_BO, PK_FFN_NORM, PK_WGU, PK_BGU, PK_WDOWN, PK_BDOWN };

static int64_t layer_numel(const OrcModelCfg* c, int k) {
    int64_t D = c->D, F = c->F;
    switch (k) {
        case PK_ATTN_NORM: return D;      case PK_WQKV: return D * 3 * D;  case PK_BQKV: return 3 * D;
        case PK_WO: return D * D;         case PK_BO: return D;            case PK_FFN_NORM: return D;
        case PK_WGU: return D * 2 * F;    case PK_BGU: return 2 * F;       case PK_WDOWN: return F * D;
        default: return D;
    }
}

static int64_t layer_total(const OrcModelCfg* c) {
    int64_t n = 0;
    for (int k = 0; k < 10; k++) n += layer_numel(c, k);
    return n;
}

static int64_t param_off(const OrcModelCfg* c, int layer, int k) {
    int64_t off = (int64_t)c->V * c->D + (int64_t)layer * layer_total(c);
    for (int i = 0; i < k; i++) off += layer_numel(c, i);
    return off;
}

int64_t orc_model_total_scalars(const OrcModelCfg* c) {
    return (int64_t)c->V * c->D + (int64_t)c->L * layer_total(c) + c->D;
}

static float* falloc(int64_t n) { return (float*)calloc((size_t)(n > 0 ? n : 1), sizeof(float)); }

static void gemm1(int ta, int tb, const float* A, const float* B, float* C, int M, int N, int K, float beta, int mode) {
    int lda = ta ? M : K, ldb = tb ? K : N;
    orc_gemm(ta, tb, A, B, C, M, N, K, lda, ldb, N, 1, 0, 0, 0, 1.0f, beta, mode);
}

typedef struct { float* S; int T; float scale; } SmJob;
static void softmax_rows(int64_t lo, int64_t hi, void* arg) {
    SmJob* j = (SmJob*)arg; int T = j->T;
    for (int64_t row = lo; row < hi; row++) {
        int i = (int)(row % T); float* s = j->S + row * T;
        float mx = -3.0e38f;
        for (int k = 0; k < T; k++) { float v = s[k] * j->scale + ((k <= i) ? 0.0f : -1e9f); s[k] = v; if (v > mx) mx = v; }
        float sum = 0.0f;
        for (int k = 0; k < T; k++) { float e = expf(s[k] - mx); s[k] = e; sum += e; }
        for (int k = 0; k < T; k++) s[k] /= sum;
    }
}

typedef struct { const float* P; float* dP; int T; float scale; } SmbJob;
static void softmax_bwd_rows(int64_t lo, int64_t hi, void* arg) {
    SmbJob* j = (SmbJob*)arg; int T = j->T;
    for (int64_t row = lo; row < hi; row++) {
        const float* p = j->P + row * T; float* d = j->dP + row * T;
        float dot = 0.0f;
        for (int k = 0; k < T; k++) dot += d[k] * p[k];
        for (int k = 0; k < T; k++) d[k] = p[k] * (d[k] - dot) * j->scale;
    }
}

typedef struct LayerActs { float *x_in, *n1, *r1, *Q, *K, *V, *P, *att, *x2, *n2, *r2, *gu, *h; } LayerActs;

float orc_model_forward_backward(const OrcModelCfg* c, const float* params,
                                 const uint32_t* ids, const uint32_t* targets,
                                 float* grads, float* logits_out, int mode, int mode_dw) {
    int V = c->V, D = c->D, H = c->H, L = c->L, F = c->F, T = c->T, B = c->B;
    int N = B * T, hd = D / H, BH = B * H;
    int64_t sTT = (int64_t)T * T, sThd = (int64_t)T * hd;
    float scale = 1.0f / sqrtf((float)hd);
    const float* E = params;
    int64_t p_final = (int64_t)V * D + (int64_t)L * layer_total(c);

    float* cos_t = falloc((int64_t)T * hd / 2); float* sin_t = falloc((int64_t)T * hd / 2);
    orc_rope_tables(T, hd, 10000.0f, cos_t, sin_t);

    LayerActs* acts = (LayerActs*)calloc((size_t)L, sizeof(LayerActs));
    float* x_final = falloc((int64_t)N * D);
    float* qkv = falloc((int64_t)N * 3 * D);
    float* Obuf = falloc((int64_t)N * D);

    /* ---- forward: model/gpu_train.c:324-384 ---- */
    for (int l = 0; l < L; l++) {
        LayerActs* a = &acts[l];
        a->x_in = falloc((int64_t)N * D); a->n1 = falloc((int64_t)N * D); a->r1 = falloc(N);
        a->Q = falloc((int64_t)N * D); a->K = falloc((int64_t)N * D); a->V = falloc((int64_t)N * D);
        a->P = falloc((int64_t)BH * sTT); a->att = falloc((int64_t)N * D); a->x2 = falloc((int64_t)N * D);
        a->n2 = falloc((int64_t)N * D); a->r2 = falloc(N); a->gu = falloc((int64_t)N * 2 * F); a->h = falloc((int64_t)N * F);
    }
    orc_embed_fwd(E, ids, L > 0 ? acts[0].x_in : x_final, N, D);
    for (int l = 0; l < L; l++) {
        LayerActs* a = &acts[l];
        float* x_out = (l + 1 < L) ? acts[l + 1].x_in : x_final;
        const float* P0 = params;
        orc_rmsnorm_fwd(a->x_in, P0 + param_off(c, l, PK_ATTN_NORM), a->n1, a->r1, N, D, c->eps);
        orc_gemm_bias(a->n1, P0 + param_off(c, l, PK_WQKV), P0 + param_off(c, l, PK_BQKV), 0, qkv, N, 3 * D, D, mode);
        orc_qkv_rope_split(qkv, cos_t, sin_t, a->Q, a->K, a->V, B, T, H, hd);
        orc_gemm(0, 1, a->Q, a->K, a->P, T, T, hd, hd, hd, T, BH, sThd, sThd, sTT, 1.0f, 0.0f, mode);
        { SmJob j = { a->P, T, scale }; parallel_for((int64_t)BH * T, softmax_rows, &j); }
        orc_gemm(0, 0, a->P, a->V, Obuf, T, hd, T, T, hd, hd, BH, sTT, sThd, sThd, 1.0f, 0.0f, mode);
        orc_heads_merge(Obuf, a->att, B, T, H, hd);
        orc_gemm_bias(a->att, P0 + param_off(c, l, PK_WO), P0 + param_off(c, l, PK_BO), a->x_in, a->x2, N, D, D, mode);
        orc_rmsnorm_fwd(a->x2, P0 + param_off(c, l, PK_FFN_NORM), a->n2, a->r2, N, D, c->eps);
        orc_gemm_bias(a->n2, P0 + param_off(c, l, PK_WGU), P0 + param_off(c, l, PK_BGU), 0, a->gu, N, 2 * F, D, mode);
        orc_swiglu_fwd(a->gu, a->h, N, F);
        orc_gemm_bias(a->h, P0 + param_off(c, l, PK_WDOWN), P0 + param_off(c, l, PK_BDOWN), a->x2, x_out, N, D, F, mode);
    }
    float* nf = falloc((int64_t)N * D); float* rf = falloc(N);
    orc_rmsnorm_fwd(x_final, params + p_final, nf, rf, N, D, c->eps);
    float* logits = falloc((int64_t)N * V);
    gemm1(0, 1, nf, E, logits, N, V, D, 0.0f, mode);
    if (logits_out) memcpy(logits_out, logits, (size_t)N * V * sizeof(float));
    float* loss_rows = falloc(N);
    orc_cross_entropy(logits, targets, loss_rows, N, V, V, 1.0f / (float)N);
    float loss_sum = 0.0f;
    for (int b = 0; b < B; b++) {
        float s = 0.0f;
        for (int t = 0; t < T; t++) s += loss_rows[(int64_t)b * T + t];
        loss_sum += s / (float)T;
    }
    float loss = loss_sum / (float)B;

    /* ---- backward: model/gpu_train.c:390-474 ---- */
    if (grads) {
        memset(grads, 0, (size_t)orc_model_total_scalars(c) * sizeof(float));
        float* dres = falloc((int64_t)N * D); float* dn = falloc((int64_t)N * D);
        float* dh = falloc((int64_t)N * F); float* dgu = falloc((int64_t)N * 2 * F);
        float* datt = falloc((int64_t)N * D); float* dO = falloc((int64_t)N * D);
        float* dQ = falloc((int64_t)N * D); float* dK = falloc((int64_t)N * D); float* dV = falloc((int64_t)N * D);
        float* dP = falloc((int64_t)BH * sTT); float* dqkv = falloc((int64_t)N * 3 * D);

        gemm1(1, 0, logits, nf, grads, V, D, N, 1.0f, mode);          /* dE += dlogits^T nf */
        gemm1(0, 0, logits, E, dn, N, D, V, 0.0f, mode);              /* dnf = dlogits E */
        orc_rmsnorm_bwd(x_final, params + p_final, rf, dn, dres, grads + p_final, N, D);

        for (int l = L - 1; l >= 0; l--) {
            LayerActs* a = &acts[l];
            float* G = grads; const float* P0 = params;
            gemm1(1, 0, a->h, dres, G + param_off(c, l, PK_WDOWN), F, D, N, 1.0f, mode_dw);
            orc_colsum_acc(dres, G + param_off(c, l, PK_BDOWN), N, D);
            gemm1(0, 1, dres, P0 + param_off(c, l, PK_WDOWN), dh, N, F, D, 0.0f, mode);
            orc_swiglu_bwd(a->gu, dh, dgu, N, F);
            gemm1(1, 0, a->n2, dgu, G + param_off(c, l, PK_WGU), D, 2 * F, N, 1.0f, mode_dw);
            orc_colsum_acc(dgu, G + param_off(c, l, PK_BGU), N, 2 * F);
            gemm1(0, 1, dgu, P0 + param_off(c, l, PK_WGU), dn, N, D, 2 * F, 0.0f, mode);
            orc_rmsnorm_bwd(a->x2, P0 + param_off(c, l, PK_FFN_NORM), a->r2, dn, dres, G + param_off(c, l, PK_FFN_NORM), N, D);

            gemm1(1, 0, a->att, dres, G + param_off(c, l, PK_WO), D, D, N, 1.0f, mode_dw);
            orc_colsum_acc(dres, G + param_off(c, l, PK_BO), N, D);
            gemm1(0, 1, dres, P0 + param_off(c, l, PK_WO), datt, N, D, D, 0.0f, mode);
            orc_heads_split(datt, dO, B, T, H, hd);
            orc_gemm(1, 0, a->P, dO, dV, T, hd, T, T, hd, hd, BH, sTT, sThd, sThd, 1.0f, 0.0f, mode);
            orc_gemm(0, 1, dO, a->V, dP, T, T, hd, hd, hd, T, BH, sThd, sThd, sTT, 1.0f, 0.0f, mode);
            { SmbJob j = { a->P, dP, T, scale }; parallel_for((int64_t)BH * T, softmax_bwd_rows, &j); }
            orc_gemm(0, 0, dP, a->K, dQ, T, hd, T, T, hd, hd, BH, sTT, sThd, sThd, 1.0f, 0.0f, mode);
            orc_gemm(1, 0, dP, a->Q, dK, T, hd, T, T, hd, hd, BH, sTT, sThd, sThd, 1.0f, 0.0f, mode);
            orc_qkv_rope_merge_bwd(dQ, dK, dV, cos_t, sin_t, dqkv, B, T, H, hd);
            gemm1(1, 0, a->n1, dqkv, G + param_off(c, l, PK_WQKV), D, 3 * D, N, 1.0f, mode_dw);
            orc_colsum_acc(dqkv, G + param_off(c, l, PK_BQKV), N, 3 * D);
            gemm1(0, 1, dqkv, P0 + param_off(c, l, PK_WQKV), dn, N, D, 3 * D, 0.0f, mode);
            orc_rmsnorm_bwd(a->x_in, P0 + param_off(c, l, PK_ATTN_NORM), a->r1, dn, dres, G + param_off(c, l, PK_ATTN_NORM), N, D);
        }
        orc_embed_bwd(dres, ids, grads, N, D);
        free(dres); free(dn); free(dh); free(dgu); free(datt); free(dO);
        free(dQ); free(dK); free(dV); free(dP); free(dqkv);
    }

    for (int l = 0; l < L; l++) {
        LayerActs* a = &acts[l];
        free(a->x_in); free(a->n1); free(a->r1); free(a->Q); free(a->K); free(a->V); free(a->P);
        free(a->att); free(a->x2); free(a->n2); free(a->r2); free(a->gu); free(a->h);
    }
    free(acts); free(x_final); free(qkv); free(Obuf); free(nf); free(rf); free(logits); free(loss_rows);
    free(cos_t); free(sin_t);
    return loss;
}
