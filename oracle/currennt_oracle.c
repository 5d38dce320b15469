/*
 * TEST INFRASTRUCTURE ONLY -- never linked into, imported by, or called from the shipped library.
 *
 * A plain-C restatement of the reference toolkit's CPU ("Cpu device") arithmetic for the LSTM
 * training path: input -> {feedforward_*, lstm, blstm}* -> sse, one forward pass, the SSE error,
 * one BPTT backward pass, all weight gradients and the steepest-descent update.  It is the
 * checker the CUDA kernels are compared with, and the timed single-thread CPU baseline when the
 * compiled reference library is not available.
 *
 * Parity status: PINNED.  The reference ships no tests or golden vectors for this path, so the
 * pin is the reference's own Cpu code compiled from its sources (oracle/build_ref.sh ->
 * oracle/_ref/libcurrennt_ref.so); tests/golden/ holds tensors produced by that library and the
 * CPU tests require this file to reproduce them (and, where the library is present, to agree with
 * it on fresh seeded inputs).
 *
 * Every loop follows the summation order of the reference so that the fp32 build agrees with it
 * to the last few ulps.  REAL may be set to double (-DREAL=double) to obtain an fp64 arbiter with
 * the same structure.
 *
 * Reference files restated (paths inside the reference project, CURRENNT_codes/currennt_lib/src/):
 *   activation_functions/Logistic.cuh:33-48, Tanh.cuh:33-41, Maxmin1.cuh:33-36
 *   helpers/limitedError.cuh:31-34, boundRange.cuh:31-34, NumericLimits.cuh:41 (expLimit)
 *   helpers/Matrix.cu:41-183 (naive column-major products, sum first, then add to the old value)
 *   layers/LstmLayer.cu:57-185 (forward cell), :237-405 (backward cell), :407-648 (gradients),
 *                       :1744-1949 (forward loops), :2067-2382 (backward loops)
 *   layers/FeedForwardLayer.cu:53-74,106-138,1061-1101,1634-1738
 *   layers/SsePostOutputLayer.cu:94-136,166-267
 *   layers/InputLayer.cu:162-164, layers/Layer.cu:254-305 (loadSequences)
 *   optimizers/SteepestDescentOptimizer.cu:74-100 (UpdateWeightFn)
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifndef REAL
#define REAL float
#endif
typedef REAL real_t;

enum { L_INPUT = 0, L_FF_TANH = 1, L_FF_LOGISTIC = 2, L_FF_IDENTITY = 3, L_LSTM = 4, L_BLSTM = 5, L_SSE = 6 };
enum { PAT_NONE = 0, PAT_FIRST = 1, PAT_NORMAL = 2, PAT_LAST = 3 }; /* Types.hpp:35-38 */

static real_t real_exp(real_t x) { return sizeof(real_t) == 4 ? (real_t)expf((float)x) : (real_t)exp((double)x); }

/* Logistic.cuh:33-43 with expLimit = 88.722839 (NumericLimits.cuh:41) */
static real_t act_logistic(real_t x) {
    const real_t lim = (real_t)88.722839;
    if (x < lim) {
        if (x > -lim) return (real_t)1.0 / ((real_t)1.0 + real_exp(-x));
        return 0;
    }
    return 1;
}
static real_t d_logistic(real_t y) { return y * ((real_t)1.0 - y); }                  /* Logistic.cuh:45-48 */
static real_t act_maxmin1(real_t x) { return (real_t)2.0 * act_logistic(x) - (real_t)1.0; } /* Maxmin1.cuh:33-36 */
static real_t act_tanh(real_t x) { return act_maxmin1((real_t)2.0 * x); }             /* Tanh.cuh:33-36 */
static real_t d_tanh(real_t y) { return (real_t)1.0 - (y * y); }                      /* Tanh.cuh:38-41 */
static real_t limited_error(real_t e) { return e < (real_t)-1.0 ? (real_t)-1.0 : (e > (real_t)1.0 ? (real_t)1.0 : e); }

typedef struct {
    real_t *ni, *ig, *fg, *og, *c, *h;      /* activations, cell states, block outputs [T*P*els] */
    real_t *dni, *dig, *dfg, *dog, *ce, *e; /* deltas, cell-state errors, output errors    */
} lstm_dir;

typedef struct {
    int type, size, prev_size;
    real_t bias;
    long nw;
    real_t *out, *err;       /* outputs / outputErrors [maxT*P*size] */
    real_t *w, *dw, *mom;    /* weights / weightUpdates / momentum deltas */
    real_t *err_in;          /* outputErrors as they were just before this layer's backward */
    lstm_dir d[2];
} layer_t;

typedef struct {
    int n, P, maxT, T, Tmin;
    layer_t *L;
    char *pat;
} net_t;

static real_t *zalloc(size_t n) { return (real_t *)calloc(n ? n : 1, sizeof(real_t)); }

long oracle_lstm_num_weights(int prev, int size, int bidir) { /* LstmLayer.cu:1085-1088 */
    int els = bidir ? size / 2 : size;
    return (long)size * (4 * ((long)prev + 1) + 4 * (long)els + 3);
}

void *oracle_create(int n_layers, const int *types, const int *sizes, const float *biases, int P, int maxT) {
    net_t *n = (net_t *)calloc(1, sizeof(net_t));
    n->n = n_layers; n->P = P; n->maxT = maxT;
    n->L = (layer_t *)calloc(n_layers, sizeof(layer_t));
    n->pat = (char *)calloc((size_t)maxT * P, 1);
    for (int i = 0; i < n_layers; ++i) {
        layer_t *l = &n->L[i];
        l->type = types[i]; l->size = sizes[i]; l->bias = biases[i];
        l->prev_size = i ? sizes[i - 1] : 0;
        size_t cnt = (size_t)maxT * P * l->size;
        l->out = zalloc(cnt); l->err = zalloc(cnt); l->err_in = zalloc(cnt);
        if (l->type >= L_FF_TANH && l->type <= L_FF_IDENTITY) l->nw = (long)l->size * (l->prev_size + 1);
        else if (l->type == L_LSTM || l->type == L_BLSTM) {
            int bi = l->type == L_BLSTM, els = bi ? l->size / 2 : l->size;
            l->nw = oracle_lstm_num_weights(l->prev_size, l->size, bi);
            size_t c2 = (size_t)maxT * P * els;
            for (int d = 0; d < (bi ? 2 : 1); ++d) {
                real_t **b = (real_t **)&l->d[d];
                for (int k = 0; k < 12; ++k) b[k] = zalloc(c2);
            }
        }
        if (l->nw) { l->w = zalloc(l->nw); l->dw = zalloc(l->nw); l->mom = zalloc(l->nw); }
    }
    return n;
}

void oracle_destroy(void *h) {
    net_t *n = (net_t *)h;
    for (int i = 0; i < n->n; ++i) {
        layer_t *l = &n->L[i];
        free(l->out); free(l->err); free(l->err_in); free(l->w); free(l->dw); free(l->mom);
        for (int d = 0; d < 2; ++d) { real_t **b = (real_t **)&l->d[d]; for (int k = 0; k < 12; ++k) free(b[k]); }
    }
    free(n->L); free(n->pat); free(n);
}

int oracle_num_layers(void *h) { return ((net_t *)h)->n; }
int oracle_layer_size(void *h, int i) { return ((net_t *)h)->L[i].size; }
long oracle_num_weights(void *h, int i) { return ((net_t *)h)->L[i].nw; }
int oracle_set_weights(void *h, int i, const float *w) {
    layer_t *l = &((net_t *)h)->L[i]; if (!l->nw) return -1;
    for (long k = 0; k < l->nw; ++k) l->w[k] = w[k];
    return 0;
}
int oracle_get_weights(void *h, int i, float *w) {
    layer_t *l = &((net_t *)h)->L[i]; if (!l->nw) return -1;
    for (long k = 0; k < l->nw; ++k) w[k] = (float)l->w[k];
    return 0;
}
int oracle_get_weight_updates(void *h, int i, float *g) {
    layer_t *l = &((net_t *)h)->L[i]; if (!l->nw) return -1;
    for (long k = 0; k < l->nw; ++k) g[k] = (float)l->dw[k];
    return 0;
}

/* Layer.cu:254-305, InputLayer.cu:162-164, PostOutputLayer.cu:285-311: take over the fraction */
int oracle_load(void *h, int T, int nSeq, const int *lens, const float *inputs, const float *targets) {
    net_t *n = (net_t *)h;
    if (T > n->maxT || nSeq > n->P) return -1;
    n->T = 0; n->Tmin = 1 << 30;
    memset(n->pat, PAT_NONE, (size_t)n->maxT * n->P);
    for (int p = 0; p < nSeq; ++p) {
        if (lens[p] > n->T) n->T = lens[p];
        if (lens[p] < n->Tmin) n->Tmin = lens[p];
        for (int t = 0; t < lens[p]; ++t)
            n->pat[(size_t)t * n->P + p] = t == 0 ? PAT_FIRST : (t == lens[p] - 1 ? PAT_LAST : PAT_NORMAL);
    }
    if (n->T > T) return -1;
    layer_t *in = &n->L[0], *post = &n->L[n->n - 1];
    size_t ci = (size_t)n->T * n->P * in->size, co = (size_t)n->T * n->P * post->size;
    for (size_t k = 0; k < ci; ++k) in->out[k] = inputs[k];
    if (post->type == L_SSE) for (size_t k = 0; k < co; ++k) post->out[k] = targets[k]; /* targets live in the post layer's outputs */
    return 0;
}

/* C(rows x cols) (+)= A^T B with A (k x rows) col-major, B (k x cols) col-major: Matrix.cu:87-131 */
static void gemm_tn(real_t *C, int ldc, const real_t *A, const real_t *B, int rows, int cols, int k, int add) {
    for (int c = 0; c < cols; ++c)
        for (int r = 0; r < rows; ++r) {
            const real_t *a = A + (size_t)r * k, *b = B + (size_t)c * k;
            real_t x = 0;
            for (int i = 0; i < k; ++i) x += a[i] * b[i];
            C[(size_t)c * ldc + r] = add ? C[(size_t)c * ldc + r] + x : x;
        }
}
/* C(rows x cols) (+)= A B with A (rows x k) col-major, B (k x cols) col-major: Matrix.cu:41-85 */
static void gemm_nn(real_t *C, const real_t *A, const real_t *B, int rows, int cols, int k, int add) {
    for (int c = 0; c < cols; ++c)
        for (int r = 0; r < rows; ++r) {
            real_t x = 0;
            for (int i = 0; i < k; ++i) x += A[(size_t)i * rows + r] * B[(size_t)c * k + i];
            C[(size_t)c * rows + r] = add ? C[(size_t)c * rows + r] + x : x;
        }
}
/* C(rows x cols) = A B^T with A (rows x k), B (cols x k) col-major: Matrix.cu:133-183 */
static void gemm_nt(real_t *C, const real_t *A, const real_t *B, int rows, int cols, int k) {
    for (int c = 0; c < cols; ++c)
        for (int r = 0; r < rows; ++r) {
            real_t x = 0;
            for (int i = 0; i < k; ++i) x += A[(size_t)i * rows + r] * B[(size_t)i * cols + c];
            C[(size_t)c * rows + r] = x;
        }
}

static real_t ff_act(int type, real_t a) {
    return type == L_FF_TANH ? act_tanh(a) : (type == L_FF_LOGISTIC ? act_logistic(a) : a);
}
static real_t ff_deriv(int type, real_t y) {
    return type == L_FF_TANH ? d_tanh(y) : (type == L_FF_LOGISTIC ? d_logistic(y) : (real_t)1.0);
}

/* FeedForwardLayer.cu:1061-1101 */
static void ff_forward(net_t *n, layer_t *l, layer_t *pl) {
    int N = n->T * n->P;
    gemm_tn(l->out, l->size, l->w, pl->out, l->size, N, pl->size, 0);
    const real_t *b = l->w + (size_t)l->size * pl->size;
    for (size_t k = 0; k < (size_t)N * l->size; ++k) l->out[k] = ff_act(l->type, l->out[k] + l->bias * b[k % l->size]);
}

/* FeedForwardLayer.cu:1634-1738, bias gradient :118-138,1517-1533 */
static void ff_backward(net_t *n, layer_t *l, layer_t *pl) {
    int N = n->T * n->P;
    for (size_t k = 0; k < (size_t)N * l->size; ++k) l->err[k] = ff_deriv(l->type, l->out[k]) * l->err[k];
    gemm_nn(pl->err, l->w, l->err, pl->size, N, l->size, 0);
    gemm_nt(l->dw, pl->out, l->err, pl->size, l->size, N);
    real_t *db = l->dw + (size_t)l->size * pl->size;
    for (int u = 0; u < l->size; ++u) {
        real_t wu = 0;
        for (int i = 0; i < N; ++i) wu += l->bias * l->err[(size_t)i * l->size + u];
        db[u] = wu;
    }
}

/* Weight-vector layout of an (b)lstm layer, LstmLayer.hpp:36-55, LstmLayer.cu:1140-1169,1238-1267 */
typedef struct { const real_t *win[4], *b[4], *wrec[4], *peep[3]; } lstm_w;
static lstm_w lstm_weights(const layer_t *l, const real_t *base, int dir) {
    lstm_w v;
    int ls = l->size, pls = l->prev_size, bi = l->type == L_BLSTM, els = bi ? ls / 2 : ls;
    for (int g = 0; g < 4; ++g) {
        v.win[g] = base + (size_t)g * ls * pls + (size_t)dir * els * pls;
        v.b[g] = base + (size_t)4 * ls * pls + (size_t)g * ls + dir * els;
        v.wrec[g] = base + (size_t)4 * ls * (pls + 1) + (size_t)g * ls * els + (size_t)dir * els * els;
    }
    for (int q = 0; q < 3; ++q) v.peep[q] = base + (size_t)4 * ls * (pls + 1) + (size_t)4 * ls * els + (size_t)q * ls + dir * els;
    return v;
}

/* LstmLayer.cu:1744-1949 with the cell of :57-185 */
static void lstm_forward(net_t *n, layer_t *l, layer_t *pl) {
    int P = n->P, T = n->T, ls = l->size, pls = pl->size, bi = l->type == L_BLSTM, els = bi ? ls / 2 : ls;
    int N = T * P, nn = P * els;
    for (int dir = 0; dir < (bi ? 2 : 1); ++dir) {
        lstm_dir *D = &l->d[dir];
        lstm_w W = lstm_weights(l, l->w, dir);
        real_t *acts[4] = {D->ni, D->ig, D->fg, D->og};
        for (int g = 0; g < 4; ++g) gemm_tn(acts[g], els, W.win[g], pl->out, els, N, pls, 0); /* :1756-1775 */
        for (int s = 0; s < T; ++s) {
            int t = dir ? T - 1 - s : s, first = s == 0;
            int prev = dir ? t + 1 : t - 1;
            if (!first)
                for (int g = 0; g < 4; ++g) /* :1826-1837 / :1895-1906 */
                    gemm_tn(acts[g] + (size_t)t * nn, els, W.wrec[g], D->h + (size_t)prev * nn, els, P, els, 1);
            int check = t >= n->Tmin;
            for (int p = 0; p < P; ++p)
                for (int j = 0; j < els; ++j) {
                    size_t idx = (size_t)t * nn + (size_t)p * els + j, pidx = (size_t)prev * nn + (size_t)p * els + j;
                    if (check && n->pat[(size_t)t * P + p] == PAT_NONE) { /* :93-100 */
                        if (dir) D->c[idx] = 0;
                        D->h[idx] = 0;
                        continue;
                    }
                    real_t ni = D->ni[idx], ig = D->ig[idx], fg = D->fg[idx], og = D->og[idx];
                    ni += l->bias * W.b[0][j]; ig += l->bias * W.b[1][j];
                    fg += l->bias * W.b[2][j]; og += l->bias * W.b[3][j];
                    if (!first) { real_t pc = D->c[pidx]; ig += pc * W.peep[0][j]; fg += pc * W.peep[1][j]; }
                    ni = act_tanh(ni); ig = act_logistic(ig); fg = act_logistic(fg);
                    D->ni[idx] = ni; D->ig[idx] = ig; D->fg[idx] = fg;
                    real_t c = ni * ig;
                    if (!first) c += D->c[pidx] * fg;
                    D->c[idx] = c;
                    og += c * W.peep[2][j];
                    og = act_logistic(og);
                    D->og[idx] = og;
                    D->h[idx] = act_tanh(c) * og;
                }
        }
        /* ResortOutputsFn :187-208 (bidirectional) / buffer swap (unidirectional) */
        for (int f = 0; f < N; ++f)
            for (int j = 0; j < els; ++j) l->out[(size_t)f * ls + dir * els + j] = D->h[(size_t)f * els + j];
    }
}

/* LstmLayer.cu:2067-2382 with the cell of :237-405 and the gradient functor of :407-648 */
static void lstm_backward(net_t *n, layer_t *l, layer_t *pl) {
    int P = n->P, T = n->T, ls = l->size, pls = pl->size, bi = l->type == L_BLSTM, els = bi ? ls / 2 : ls;
    int N = T * P, nn = P * els, nd = bi ? 2 : 1;
    for (int dir = 0; dir < nd; ++dir) {
        lstm_dir *D = &l->d[dir];
        lstm_w W = lstm_weights(l, l->w, dir);
        real_t *dl[4] = {D->dni, D->dig, D->dfg, D->dog};
        for (int f = 0; f < N; ++f) /* ResortOutputErrorsFn :210-235 */
            for (int j = 0; j < els; ++j) D->e[(size_t)f * els + j] = l->err[(size_t)f * ls + dir * els + j];
        for (int s = 0; s < T; ++s) {
            int t = dir ? s : T - 1 - s, firstCall = s == 0, lastCall = s == T - 1;
            int next = dir ? t - 1 : t + 1, prevc = dir ? t + 1 : t - 1;
            if (!firstCall)
                for (int g = 0; g < 4; ++g) /* :2136-2147 / :2214-2225 */
                    gemm_nn(D->e + (size_t)t * nn, W.wrec[g], dl[g] + (size_t)next * nn, els, P, els, 1);
            int check = t >= n->Tmin;
            for (int p = 0; p < P; ++p)
                for (int j = 0; j < els; ++j) {
                    size_t idx = (size_t)t * nn + (size_t)p * els + j, nidx = (size_t)next * nn + (size_t)p * els + j;
                    if (check && n->pat[(size_t)t * P + p] == PAT_NONE) { /* :273-283 */
                        D->dni[idx] = D->dig[idx] = D->dfg[idx] = D->dog[idx] = 0; D->ce[idx] = 0;
                        continue;
                    }
                    real_t e = D->e[idx], ni = D->ni[idx], ig = D->ig[idx], og = D->og[idx], c = D->c[idx];
                    /* the stored og delta buffer is zero at this point for a plain LSTM (:1531) */
                    real_t dog = (d_logistic(og) * act_tanh(c) * e) + (real_t)0;
                    real_t ce = og * d_tanh(act_tanh(c)) * e + W.peep[2][j] * dog;
                    if (!firstCall)
                        ce += (D->fg[nidx] * D->ce[nidx] + W.peep[0][j] * D->dig[nidx] + W.peep[1][j] * D->dfg[nidx]);
                    real_t dni = ig * d_tanh(ni) * ce;
                    real_t dfg = 0;
                    if (!lastCall) dfg = d_logistic(D->fg[idx]) * D->c[(size_t)prevc * nn + (size_t)p * els + j] * ce;
                    real_t dig = d_logistic(ig) * ni * ce;
                    D->dni[idx] = limited_error(dni); D->dig[idx] = limited_error(dig);
                    D->dfg[idx] = limited_error(dfg); D->dog[idx] = limited_error(dog);
                    D->ce[idx] = ce;
                }
        }
    }
    /* a unidirectional layer works in place on its own outputErrors (buffer swap, :2086-2087,2378-2381),
       so after the pass that vector holds the accumulated e_t rather than what the next layer wrote */
    if (!bi) memcpy(l->err, l->d[0].e, (size_t)N * els * sizeof(real_t));
    /* error to the preceding layer, :2298-2334: assign with fw/ni, then add the other seven */
    int first = 1;
    for (int dir = 0; dir < nd; ++dir) {
        lstm_dir *D = &l->d[dir];
        lstm_w W = lstm_weights(l, l->w, dir);
        real_t *dl[4] = {D->dni, D->dig, D->dfg, D->dog};
        for (int g = 0; g < 4; ++g) { gemm_nn(pl->err, W.win[g], dl[g], pls, N, els, !first); first = 0; }
    }
    /* weight updates, :407-648: one sequential dot product over the patterns per weight */
    for (int dir = 0; dir < nd; ++dir) {
        lstm_dir *D = &l->d[dir];
        lstm_w G = lstm_weights(l, l->dw, dir);
        real_t *dl[4] = {D->dni, D->dig, D->dfg, D->dog};
        int skip = P;                       /* patterns of one timestep */
        for (int g = 0; g < 4; ++g) {
            real_t *gin = (real_t *)G.win[g], *gb = (real_t *)G.b[g], *grec = (real_t *)G.wrec[g];
            for (int j = 0; j < els; ++j) {
                for (int i = 0; i < pls; ++i) { /* input weights :490-522 */
                    real_t wu = 0;
                    for (int f = 0; f < N; ++f) wu += pl->out[(size_t)f * pls + i] * dl[g][(size_t)f * els + j];
                    gin[(size_t)j * pls + i] = wu;
                }
                { /* bias :524-541 */
                    real_t wu = 0;
                    for (int f = 0; f < N; ++f) wu += l->bias * dl[g][(size_t)f * els + j];
                    gb[j] = wu;
                }
                for (int k = 0; k < els; ++k) { /* recurrent :543-572,629-636 */
                    real_t wu = 0;
                    if (!dir) for (int f = skip; f < N; ++f) wu += D->h[(size_t)(f - skip) * els + k] * dl[g][(size_t)f * els + j];
                    else      for (int f = 0; f < N - skip; ++f) wu += D->h[(size_t)(f + skip) * els + k] * dl[g][(size_t)f * els + j];
                    grec[(size_t)j * els + k] = wu;
                }
            }
        }
        for (int q = 0; q < 3; ++q) { /* peepholes :574-610: ig, fg use the other step's cell state, og the same step's */
            real_t *gp = (real_t *)G.peep[q];
            for (int j = 0; j < els; ++j) {
                real_t wu = 0;
                if (q == 2) for (int f = 0; f < N; ++f) wu += D->c[(size_t)f * els + j] * dl[3][(size_t)f * els + j];
                else if (!dir) for (int f = skip; f < N; ++f) wu += D->c[(size_t)(f - skip) * els + j] * dl[q + 1][(size_t)f * els + j];
                else for (int f = 0; f < N - skip; ++f) wu += D->c[(size_t)(f + skip) * els + j] * dl[q + 1][(size_t)f * els + j];
                gp[j] = wu;
            }
        }
    }
}

/* forward through all layers; returns the SSE of SsePostOutputLayer.cu:94-116,197-209 */
double oracle_forward(void *h) {
    net_t *n = (net_t *)h;
    for (int i = 1; i < n->n; ++i) {
        layer_t *l = &n->L[i], *pl = &n->L[i - 1];
        if (l->type >= L_FF_TANH && l->type <= L_FF_IDENTITY) ff_forward(n, l, pl);
        else if (l->type == L_LSTM || l->type == L_BLSTM) lstm_forward(n, l, pl);
    }
    layer_t *post = &n->L[n->n - 1], *pl = &n->L[n->n - 2];
    if (post->type != L_SSE) return 0;
    real_t s = 0;
    size_t cnt = (size_t)n->T * n->P * post->size;
    for (size_t k = 0; k < cnt; ++k) {
        if (n->pat[k / post->size] == PAT_NONE) continue;
        real_t d = post->out[k] - pl->out[k];
        s += d * d;
    }
    return (double)((real_t)0.5 * s);
}

void oracle_backward(void *h) {
    net_t *n = (net_t *)h;
    for (int i = n->n - 1; i >= 1; --i) {
        layer_t *l = &n->L[i], *pl = &n->L[i - 1];
        size_t cnt = (size_t)n->T * n->P * l->size;
        memcpy(l->err_in, l->err, cnt * sizeof(real_t));
        if (l->type == L_SSE) { /* SsePostOutputLayer.cu:118-136,255-265: writes the preceding layer's errors */
            for (size_t k = 0; k < cnt; ++k)
                pl->err[k] = n->pat[k / l->size] == PAT_NONE ? 0 : pl->out[k] - l->out[k];
        } else if (l->type >= L_FF_TANH && l->type <= L_FF_IDENTITY) ff_backward(n, l, pl);
        else if (l->type == L_LSTM || l->type == L_BLSTM) lstm_backward(n, l, pl);
    }
}

static long copy_out(net_t *n, int i, const real_t *src, float *dst) {
    size_t cnt = (size_t)n->T * n->P * n->L[i].size;
    for (size_t k = 0; k < cnt; ++k) dst[k] = (float)src[k];
    return (long)cnt;
}
long oracle_get_outputs(void *h, int i, float *o) { net_t *n = (net_t *)h; return copy_out(n, i, n->L[i].out, o); }
long oracle_get_output_errors(void *h, int i, float *o) { net_t *n = (net_t *)h; return copy_out(n, i, n->L[i].err, o); }
long oracle_get_output_errors_in(void *h, int i, float *o) { net_t *n = (net_t *)h; return copy_out(n, i, n->L[i].err_in, o); }

/* SteepestDescentOptimizer.cu:74-100: g<-0 if NaN/Inf; delta<-mom*delta-lr*g; w<-w+delta */
void oracle_sgd_update(void *h, float lr, float mom) {
    net_t *n = (net_t *)h;
    for (int i = 0; i < n->n; ++i) {
        layer_t *l = &n->L[i];
        for (long k = 0; k < l->nw; ++k) {
            real_t g = l->dw[k];
            if (isnan(g) || isinf(g)) { g = 0; l->dw[k] = 0; }
            real_t d = (real_t)mom * l->mom[k] - (real_t)lr * g;
            l->mom[k] = d;
            l->w[k] = l->w[k] + d;
        }
    }
}
