/* CPU oracle: exact k-class Jenks natural breaks -- TEST INFRASTRUCTURE ONLY.
 *
 * Restates, for k classes, the objective the reference evaluates for two
 * classes in Python_Jenks_Test/Jenks_Tests/cuda_helpers.py:151-184 (host
 * wrapper :378-395): over the ascending-sorted values choose contiguous
 * classes that minimise the total within-class sum of squared deviations,
 * the first minimum winning.  The reference has no k>2 source and its k=2
 * kernel is O(n^2) per candidate; this is the textbook Fisher-Jenks dynamic
 * programme in its plain O(k m^2) form, kept deliberately simple so that it
 * can serve as the definition the faster product implementations are
 * checked against.  Parity unpinned: the reference holds no golden vectors.
 *
 * Input is the run-length-compressed sorted row: m distinct ascending values
 * v[] with multiplicities cnt[].  All arithmetic is IEEE double, evaluated in
 * the order written (compile with -ffp-contract=off).
 *
 *   P1[i] = sum_{t<i} cnt[t]*v[t]      P2[i] = sum_{t<i} (cnt[t]*v[t])*v[t]
 *   C[i]  = sum_{t<i} cnt[t]
 *   cost(a,b) = (P2[b]-P2[a]) - ((P1[b]-P1[a])*(P1[b]-P1[a])) / (C[b]-C[a])
 *   D[1][i] = cost(0,i)
 *   D[j][i] = min_{j-1 <= t < i} D[j-1][t] + cost(t,i), smallest t on ties
 *
 * breaks[0..k] receives 0 = b_0 < b_1 < ... < b_k = m; class c covers the
 * distinct values b_c .. b_{c+1}-1.  Returns the number of classes used,
 * min(k, m), or -1 on allocation failure.
 */
#include <stdlib.h>
#include <string.h>
#include <float.h>

static double seg_cost(const double *P1, const double *P2, const double *C, int a, int b)
{
    double d1 = P1[b] - P1[a];
    double d2 = P2[b] - P2[a];
    double c = C[b] - C[a];
    double sq = d1 * d1;
    double q = sq / c;
    return d2 - q;
}

int jq_oracle_jenks_breaks(const double *v, const double *cnt, int m, int k, int *breaks)
{
    if (m <= 0 || k <= 0) return 0;
    int ke = k < m ? k : m;
    double *P1 = (double *)malloc(sizeof(double) * (size_t)(m + 1) * 5);
    int *arg = (int *)malloc(sizeof(int) * (size_t)(m + 1) * (size_t)(ke + 1));
    if (!P1 || !arg) { free(P1); free(arg); return -1; }
    double *P2 = P1 + (m + 1), *C = P2 + (m + 1), *prev = C + (m + 1), *cur = prev + (m + 1);
    P1[0] = 0.0; P2[0] = 0.0; C[0] = 0.0;
    for (int t = 0; t < m; ++t) {
        double cv = cnt[t] * v[t];
        double cvv = cv * v[t];
        P1[t + 1] = P1[t] + cv;
        P2[t + 1] = P2[t] + cvv;
        C[t + 1] = C[t] + cnt[t];
    }
    for (int i = 0; i <= m; ++i) { prev[i] = DBL_MAX; cur[i] = DBL_MAX; }
    for (int i = 1; i <= m; ++i) { prev[i] = seg_cost(P1, P2, C, 0, i); arg[1 * (m + 1) + i] = 0; }
    for (int j = 2; j <= ke; ++j) {
        for (int i = 0; i <= m; ++i) cur[i] = DBL_MAX;
        for (int i = j; i <= m; ++i) {
            double best = DBL_MAX; int bt = j - 1;
            for (int t = j - 1; t < i; ++t) {
                double c = prev[t] + seg_cost(P1, P2, C, t, i);
                if (c < best) { best = c; bt = t; }
            }
            cur[i] = best;
            arg[j * (m + 1) + i] = bt;
        }
        double *tmp = prev; prev = cur; cur = tmp;
    }
    breaks[ke] = m;
    for (int j = ke; j >= 1; --j) breaks[j - 1] = arg[j * (m + 1) + breaks[j]];
    free(P1); free(arg);
    return ke;
}

/* Same DP evaluated by exhaustive enumeration of all break sets: only for
 * m <= ~14.  Ties go to the lexicographically smallest break vector when
 * compared from the LAST break backwards, which is what the DP's backtrack
 * (smallest t at the final stage first) produces. */
static void brute_rec(const double *P1, const double *P2, const double *C, int m, int ke,
                      int depth, int *cur, double *best, int *bestb)
{
    if (depth == ke) {
        if (cur[ke] != m) return;
        /* evaluate in DP association order: ((c1 + c2) + c3) + ... */
        double tot = seg_cost(P1, P2, C, cur[0], cur[1]);
        for (int c = 1; c < ke; ++c) tot = tot + seg_cost(P1, P2, C, cur[c], cur[c + 1]);
        int better = 0;
        if (tot < *best) better = 1;
        else if (tot == *best) {
            for (int c = ke - 1; c >= 1; --c) {
                if (cur[c] != bestb[c]) { better = cur[c] < bestb[c]; break; }
            }
        }
        if (better) { *best = tot; memcpy(bestb, cur, sizeof(int) * (size_t)(ke + 1)); }
        return;
    }
    int lo = cur[depth] + 1;
    int hi = (depth == ke - 1) ? m : m - (ke - 1 - depth);
    if (depth == ke - 1) lo = m;
    for (int b = lo; b <= hi; ++b) { cur[depth + 1] = b; brute_rec(P1, P2, C, m, ke, depth + 1, cur, best, bestb); }
}

int jq_oracle_jenks_brute(const double *v, const double *cnt, int m, int k, int *breaks)
{
    if (m <= 0 || k <= 0) return 0;
    int ke = k < m ? k : m;
    double *P1 = (double *)malloc(sizeof(double) * (size_t)(m + 1) * 3);
    if (!P1) return -1;
    double *P2 = P1 + (m + 1), *C = P2 + (m + 1);
    P1[0] = P2[0] = C[0] = 0.0;
    for (int t = 0; t < m; ++t) {
        double cv = cnt[t] * v[t];
        double cvv = cv * v[t];
        P1[t + 1] = P1[t] + cv; P2[t + 1] = P2[t] + cvv; C[t + 1] = C[t] + cnt[t];
    }
    int cur[64], bestb[64];
    double best = DBL_MAX;
    if (ke + 1 > 64) { free(P1); return -1; }
    for (int c = 0; c <= ke; ++c) bestb[c] = 0x7fffffff;
    cur[0] = 0;
    brute_rec(P1, P2, C, m, ke, 0, cur, &best, bestb);
    for (int c = 0; c <= ke; ++c) breaks[c] = bestb[c];
    free(P1);
    return ke;
}
