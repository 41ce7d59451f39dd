// Augmented-Lagrangian row laws in float, as used by the reference's tile solver:
// src/nk/solve/augmented_row.hpp:231-251 (scalar), :319-363 (friction cone), :111-138 (secant relaxation)
// and the dual helpers of ops/block_descent.cu:759-820.
#pragma once
#include "nkb_math.cuh"

namespace nkb {

struct Resp { float dual_scale, residual_scale; };
struct STerm { float impulse, curvature; };

NKB_DEV Resp scalar_response(float cap, float compliance) {
    const float product = cap * compliance;
    Resp r;
    if (product >= 1.0f) { r.dual_scale = 0.0f; r.residual_scale = 1.0f / compliance; }
    else { r.dual_scale = 1.0f - product; r.residual_scale = cap; }
    return r;
}

NKB_DEV STerm scalar_impulse(float dual, float rho, float residual, float lower, float upper, Resp rs) {
    STerm t; t.impulse = 0.f; t.curvature = 0.f;
    if (rho <= 0.0f) return t;
    if (dual != dual || rho != rho || residual != residual || lower != lower || upper != upper) {
        const float invalid = dual + rho + residual + lower + upper;
        t.impulse = t.curvature = invalid;
        return t;
    }
    const float k = rs.residual_scale;
    const float x = fmaf(k, residual, rs.dual_scale * dual);
    t.impulse = x < lower ? lower : (x > upper ? upper : x);
    t.curvature = x != x ? x : (lower < upper && x >= lower && x <= upper ? k : 0.0f);
    return t;
}

// The reference's cone argument (augmented_row.hpp:319-340) at a normalised coefficient of 1: compensated
// dual + rho * residual, no divisions
NKB_DEV float cone_argument_unit(float dual, float rho, float residual) {
    const float t = __fmul_rn(rho, residual);
    const float t_low = fmaf(rho, residual, -t);
    const float sum = __fadd_rn(dual, t);
    const float t_part = __fsub_rn(sum, dual);
    const float sum_low = __fadd_rn(__fsub_rn(dual, __fsub_rn(sum, t_part)), __fsub_rn(t, t_part));
    return __fadd_rn(sum, __fadd_rn(sum_low, t_low));
}

// Impulse (y, z) and curvature (yy, zz, yz) of the friction rows at a fixed cone radius (augmented_row.hpp:341-363)
// for one isotropic friction coefficient: the reference's projection without the per-axis scaling, the direction
// normalised by a reciprocal square root.  Invalid inputs propagate as NaN through the arithmetic.
NKB_DEV void cone_impulse(V3 dual, float rho, float res_y, float res_z, float normal_impulse, float mu,
                          float& iy, float& iz, float& cyy, float& czz, float& cyz) {
    iy = iz = cyy = czz = cyz = 0.f;
    if (rho <= 0.0f || mu <= 0.0f) return;
    const float q_y = cone_argument_unit(dual.y, rho, res_y), q_z = cone_argument_unit(dual.z, rho, res_z);
    const float radius = (normal_impulse < 0.0f ? 0.0f : normal_impulse) * mu;
    if (radius == 0.0f) return;
    const float n2 = fmaf(q_y, q_y, q_z * q_z);
    if (n2 <= radius * radius) { iy = q_y; iz = q_z; cyy = czz = rho; return; }
    const float inv = rsqrtf(n2);
    const float dy = q_y * inv, dz = q_z * inv, cs = rho * radius * inv;
    iy = radius * dy; iz = radius * dz;
    cyy = cs * dz * dz; czz = cs * dy * dy; cyz = -cs * dy * dz;
}

// ---- dual update helpers (ops/block_descent.cu:759-820) for one friction coefficient per contact: the reference's
// per-axis coefficients are both mu in this library, so its normalised coefficients are 1 and the divisions drop out ----
struct Relax { V3 step; float weight; V3 point; };
NKB_DEV V3 relax_contact_impulse_fast(V3 dual, V3 next, Relax& last) {
    const V3 step = next - dual;
    const V3 change = step - last.step;
    const V3 moved = dual - last.point;
    const float square = change.x * change.x + change.y * change.y + change.z * change.z;
    const float along = -(moved.x * change.x + moved.y * change.y + moved.z * change.z);
    float weight = 1.0f;
    if (last.weight > 0.0f && along > 0.0f && square > 0.0f) weight = fminf(1.0f, __fdividef(along, square));
    last.step = step; last.weight = weight; last.point = dual;
    return mk3(dual.x + weight * step.x, dual.y + weight * step.y, dual.z + weight * step.z);
}
NKB_DEV void multiplier_steps_iso(V3 dual, V3 next, float scale, float dual_scale, float rho, float mu, float& normal, float& tangent) {
    normal = scale > 0.0f && dual_scale != 0.0f ? __fdividef(fabsf(next.x - dual.x), scale) : 0.0f;
    const float dy = next.y - dual.y, dz = next.z - dual.z;
    tangent = mu > 0.0f && rho > 0.0f ? __fdividef(sqrtf(fmaf(dy, dy, dz * dz)), rho) : 0.0f;
}
// sum over axes of (point - next)(next - base) / metric, metric = (scale, rho, rho) for a cone head with mu > 0
NKB_DEV double momentum_restart_iso(V3 point, V3 next, V3 base, float scale, float rho, bool cone) {
    double r = 0.0;
    if (scale > 0.0f) r += ((double)point.x - next.x) * ((double)next.x - base.x) * (double)__frcp_rn(scale);
    if (cone && rho > 0.0f)
        r += (((double)point.y - next.y) * ((double)next.y - base.y) + ((double)point.z - next.z) * ((double)next.z - base.z)) * (double)__frcp_rn(rho);
    return r;
}
NKB_DEV V3 extrapolate_dual_iso(V3 base, V3 next, float beta, float lower, float upper, bool contact, float mu) {
    if (beta == 0.0f) return next;
    V3 y = mk3(fmaf(beta, next.x - base.x, next.x), fmaf(beta, next.y - base.y, next.y), fmaf(beta, next.z - base.z, next.z));
    y.x = fminf(fmaxf(y.x, lower), upper);
    if (!contact) return mk3(y.x, 0.0f, 0.0f);
    if (!(mu > 0.0f)) return mk3(y.x, 0.0f, 0.0f);
    const float s2 = fmaf(y.y, y.y, y.z * y.z), limit = fmaxf(y.x, 0.0f) * mu;
    const float scale = s2 > limit * limit ? limit * rsqrtf(s2) : 1.0f;
    return mk3(y.x, y.y * scale, y.z * scale);
}

NKB_DEV float along_axis(float impulse, float velocity) { return impulse > 0.0f ? velocity : impulse < 0.0f ? -velocity : 0.0f; }
NKB_DEV float residual_abs(float v) { return v <= FLT_MAX ? fabsf(v) : FLT_MAX; }

}  // namespace nkb
