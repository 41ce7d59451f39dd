/* Oracle (test infrastructure): augmented-Lagrangian row laws in float.
 * Restates the reference's src/nk/solve/augmented_row.hpp (float variants used by the tile route)
 * and the dual helpers of ops/block_descent.cu:759-820. */
#ifndef ORC_LAWS_H
#define ORC_LAWS_H
#include "orc_math.h"

typedef struct { float dual_scale, residual_scale; } resp_t;
typedef struct { float impulse, curvature; } sterm_t;
typedef struct { float xx, yy, zz, xy, xz, yz; } sym3;

/* augmented_row.hpp:231-234 */
static inline resp_t float_scalar_response(float cap, float compliance) {
    const float product = cap * compliance;
    resp_t r;
    if (product >= 1.0f) { r.dual_scale = 0.0f; r.residual_scale = 1.0f / compliance; }
    else { r.dual_scale = 1.0f - product; r.residual_scale = cap; }
    return r;
}

/* augmented_row.hpp:237-251 EvaluateScalarImpulse (float response) */
static inline sterm_t scalar_impulse(float dual, float rho, float residual, float compliance, float lower, float upper, resp_t rs) {
    sterm_t t = {0.0f, 0.0f};
    if (rho <= 0.0f) return t;
    if (dual != dual || rho != rho || residual != residual || compliance != compliance || lower != lower || upper != upper) {
        const float invalid = dual + rho + residual + compliance + lower + upper;
        t.impulse = t.curvature = invalid;
        return t;
    }
    const float k = rs.residual_scale;
    const float x = fmaf(k, residual, rs.dual_scale * dual);
    t.impulse = x < lower ? lower : (x > upper ? upper : x);
    t.curvature = x != x ? x : (lower < upper && x >= lower && x <= upper ? k : 0.0f);
    return t;
}

/* augmented_row.hpp:319-334 ConeArgument */
static inline float cone_argument(float dual, float rho, float mu, float residual) {
    const int dual_zero = dual == 0.0f;
    const float dual_quotient = (dual + (float)dual_zero) / mu;
    const float d = dual_zero ? dual : dual_quotient;
    const float low = fmaf(-d, mu, dual);
    const int low_zero = low == 0.0f;
    const float low_quotient = (low + (float)low_zero) / mu;
    const float d_low = low_zero ? low : low_quotient;
    volatile float p = rho * mu;
    volatile float t = p * residual;
    const float t_low = fmaf(p, residual, -t) + fmaf(rho, mu, -p) * residual;
    volatile float sum = d + t;
    volatile float t_part = sum - d;
    const float sum_low = (d - (sum - t_part)) + (t - t_part);
    return sum + (sum_low + d_low + t_low);
}

/* augmented_row.hpp:337-363 EvaluateTangentImpulse: impulse (y,z) and curvature (yy,zz,yz) */
static inline void tangent_impulse(v3 dual, float rho, v3 residual, float normal_impulse, float mu_first, float mu_second,
                                   v3 *impulse, sym3 *curv) {
    *impulse = V3(0, 0, 0);
    sym3 z = {0, 0, 0, 0, 0, 0};
    *curv = z;
    if (rho <= 0.0f) return;
    const float scale = fmaxf(mu_first, mu_second);
    const float mu_y = mu_first <= 0.0f ? 0.0f : mu_first / scale;
    const float mu_z = mu_second <= 0.0f ? 0.0f : mu_second / scale;
    const float q_y = mu_y == 0.0f ? 0.0f : cone_argument(dual.y, rho, mu_y, residual.y);
    const float q_z = mu_z == 0.0f ? 0.0f : cone_argument(dual.z, rho, mu_z, residual.z);
    const float radius = (normal_impulse < 0.0f ? 0.0f : normal_impulse) * fmaxf(scale, 0.0f);
    if (q_y != q_y || q_z != q_z || radius != radius || rho != rho) {
        const float invalid = q_y + q_z + radius + rho;
        *impulse = V3(0.0f, invalid, invalid);
        curv->yy = curv->zz = curv->yz = invalid;
        return;
    }
    if (radius == 0.0f) return;
    const float norm = hypotf(q_y, q_z);
    if (norm <= radius) {
        *impulse = V3(0.0f, mu_y * q_y, mu_z * q_z);
        curv->yy = rho * mu_y * mu_y; curv->zz = rho * mu_z * mu_z;
        return;
    }
    const float dy = q_y / norm, dz = q_z / norm, cs = rho * radius / norm;
    *impulse = V3(0.0f, mu_y * radius * dy, mu_z * radius * dz);
    curv->yy = cs * mu_y * mu_y * dz * dz;
    curv->zz = cs * mu_z * mu_z * dy * dy;
    curv->yz = -cs * mu_y * mu_z * dy * dz;
}

/* augmented_row.hpp:111-138 */
typedef struct { v3 step; float weight; v3 point; } relax_t;
static inline v3 relax_contact_impulse(v3 dual, v3 next, relax_t *last) {
    const v3 step = vsub(next, dual);
    const v3 change = vsub(step, last->step);
    const v3 moved = vsub(dual, last->point);
    const float square = change.x * change.x + change.y * change.y + change.z * change.z;
    const float along = -(moved.x * change.x + moved.y * change.y + moved.z * change.z);
    float weight = 1.0f;
    if (last->weight > 0.0f && along > 0.0f && square > 0.0f) weight = fminf(1.0f, along / square);
    last->step = step; last->weight = weight; last->point = dual;
    return V3(dual.x + weight * step.x, dual.y + weight * step.y, dual.z + weight * step.z);
}

/* augmented_row.hpp:119-124 */
static inline double momentum_restart(v3 point, v3 next, v3 base, v3 scale) {
    return (scale.x > 0.0f ? ((double)point.x - next.x) * ((double)next.x - base.x) / scale.x : 0.0) +
           (scale.y > 0.0f ? ((double)point.y - next.y) * ((double)next.y - base.y) / scale.y : 0.0) +
           (scale.z > 0.0f ? ((double)point.z - next.z) * ((double)next.z - base.z) / scale.z : 0.0);
}

/* block_descent.cu:761-770 */
static inline void multiplier_steps(v3 dual, v3 next, float scale, float dual_scale, float rho, float mu1, float mu2, float *normal, float *tangent) {
    *normal = scale > 0.0f && dual_scale != 0.0f ? fabsf(next.x - dual.x) / scale : 0.0f;
    const float fs = fmaxf(mu1, mu2);
    mu1 = mu1 <= 0.0f ? 0.0f : mu1 / fs;
    mu2 = mu2 <= 0.0f ? 0.0f : mu2 / fs;
    const float first = mu1 > 0.0f && rho > 0.0f ? (next.y - dual.y) / (rho * mu1 * mu1) : 0.0f;
    const float second = mu2 > 0.0f && rho > 0.0f ? (next.z - dual.z) / (rho * mu2 * mu2) : 0.0f;
    *tangent = hypotf(first, second);
}
/* block_descent.cu:773-775 */
static inline float along_axis(float impulse, float velocity) { return impulse > 0.0f ? velocity : impulse < 0.0f ? -velocity : 0.0f; }
/* block_descent.cu:790-795 */
static inline v3 multiplier_metric(float scale, float rho, int contact, float mu1, float mu2) {
    const float fr = fmaxf(mu1, mu2);
    const float first = contact && mu1 > 0.0f ? mu1 / fr : 0.0f;
    const float second = contact && mu2 > 0.0f ? mu2 / fr : 0.0f;
    return V3(scale, rho * first * first, rho * second * second);
}
/* block_descent.cu:808-820 */
static inline v3 extrapolate_dual(v3 base, v3 next, float beta, float lower, float upper, int contact, float mu1, float mu2) {
    if (beta == 0.0f) return next;
    v3 y = V3(fmaf(beta, next.x - base.x, next.x), fmaf(beta, next.y - base.y, next.y), fmaf(beta, next.z - base.z, next.z));
    y.x = fminf(fmaxf(y.x, lower), upper);
    if (!contact) return V3(y.x, 0.0f, 0.0f);
    const float first = mu1 > 0.0f ? y.y / mu1 : 0.0f, second = mu2 > 0.0f ? y.z / mu2 : 0.0f;
    const float slip = hypotf(first, second), radius = fmaxf(y.x, 0.0f);
    const float scale = slip > radius ? radius / slip : 1.0f;
    return V3(y.x, mu1 > 0.0f ? y.y * scale : 0.0f, mu2 > 0.0f ? y.z * scale : 0.0f);
}
static inline float residual_abs(float v) { return v <= FLT_MAX ? fabsf(v) : FLT_MAX; }

#endif
