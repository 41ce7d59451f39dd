/* Oracle (test infrastructure): the block-descent velocity solve and split-impulse position pass of one env.
 * Restates the reference's "tile route" (ops/block_descent_tile.cuh DescendTile and callees, ops/block_descent.cu
 * dual helpers, ops/block_descent_rigid.cuh) as a sequential program: blocks are the env's free bodies (6
 * coordinates: linear then angular) followed by its articulation (one coordinate per DoF); heads are the
 * active non-tangent rows in row order. */
#include <stdlib.h>
#include "orc.h"
#include "orc_math.h"
#include "orc_laws.h"

#define NO_BLOCK 0xffffffffu
#define NEWTON_STEPS 16u          /* block_descent_dense.cuh:14 */
#define LINE_STEPS 32u            /* block_descent_dense.cuh:15 */
#define LINE_TOL 1.0e-6f          /* block_descent_dense.cuh:17 */
#define ROUNDINGS 8.0f            /* block_descent_dense.cuh:19 */

void orc_factor_mass(const float *M, float *F, uint32_t n);
void orc_solve_mass(const float *F, float *x, uint32_t n);

typedef struct {
    uint32_t row, stride, axes, owner[2];
    float rho, compliance, lower, upper, mu1, mu2, normal_bound;
    resp_t rs;
    v3 dual, base, residual, move, step;
    relax_t rx;
    float *jac[2];                /* [axes][dim] per incidence */
    uint32_t flags;
} head_t;

typedef struct {
    uint32_t dim;
    float *mass;                  /* dim x dim */
    float *free_v, *vel, *pseudo;
    uint32_t color;
    uint32_t *inc; uint32_t ninc; /* incident heads in head order */
} block_t;

typedef struct {
    const orc_model *m; orc_env *e;
    head_t *heads; uint32_t nheads;
    block_t *blocks; uint32_t nblocks;
    uint32_t iteration;
    float momentum, residual;
    float tol;
} tile_t;

static float comp3(v3 v, uint32_t k) { return k == 0 ? v.x : k == 1 ? v.y : v.z; }
static void setc3(v3 *v, uint32_t k, float x) { if (k == 0) v->x = x; else if (k == 1) v->y = x; else v->z = x; }

static uint32_t side_block(const tile_t *t, const orc_side *s) {
    /* block_descent_tile.cuh:606-611 TileOwner */
    if (s->kind == ORC_SIDE_RIGID && t->blocks[s->index].dim != 0u) return s->index;
    if (s->kind == ORC_SIDE_ARTIC && t->blocks[t->m->B].dim != 0u) return t->m->B;
    return NO_BLOCK;
}

/* block_descent_tile.cuh:555-573 TileBlock::Jacobian */
static float block_jacobian(const tile_t *t, uint32_t block, const orc_row *row, uint32_t i) {
    float v = 0.0f;
    if (block < t->m->B) {
        const orc_side *sides[2] = {&row->a, &row->b};
        for (int k = 0; k < 2; ++k)
            if (sides[k]->kind == ORC_SIDE_RIGID && sides[k]->index == block)
                v += i < 3u ? sides[k]->jlin[i] : sides[k]->jang[i - 3u];
    } else {
        if (row->a.kind == ORC_SIDE_ARTIC && row->ja) v += row->ja[i];
        if (row->b.kind == ORC_SIDE_ARTIC && row->jb) v += row->jb[i];
    }
    return v;
}

/* articulation_mass.cuh:413-441 MassCoupling<float>: J A^-1 J^T from one forward solve */
static float mass_coupling(const float *F, uint32_t n, const float *v, const float *extra) {
    float y[ORC_MAX_DOF];
    for (uint32_t i = 0; i < n; ++i) {
        float a = v[i] + (extra ? extra[i] : 0.0f);
        for (uint32_t j = 0; j < i; ++j) a -= F[i * n + j] * y[j];
        y[i] = a;
    }
    float r = 0.0f;
    for (uint32_t i = 0; i < n; ++i) r += y[i] * y[i] / F[i * n + i];
    return r;
}

/* block_descent_tile.cuh:709-739 TileInertialResponse */
static float inertial_response(const tile_t *t, const orc_row *row, float *coupling, float *largest) {
    const orc_side *sides[2] = {&row->a, &row->b};
    const int shared = row->a.kind == row->b.kind && row->a.index == row->b.index;
    float response = 0.0f, shares[2] = {0.0f, 0.0f};
    int valid = 1;
    for (int i = 0; i < (shared ? 1 : 2); ++i) {
        const orc_side *s = sides[i];
        float c = 0.0f;
        if (s->kind == ORC_SIDE_RIGID) {
            v3 lin = shared ? vadd(v3ld(s->jlin), v3ld(row->b.jlin)) : v3ld(s->jlin);
            v3 ang = shared ? vadd(v3ld(s->jang), v3ld(row->b.jang)) : v3ld(s->jang);
            c = t->m->inv_mass[s->index] * vdot(lin, lin) + vdot(ang, sym_mulv(t->e->body_winv + 6 * s->index, ang));
        } else if (s->kind == ORC_SIDE_ARTIC) {
            const float *j = i == 0 ? row->ja : row->jb;
            c = mass_coupling(t->e->Mfactor, t->m->ndof, j, shared ? row->jb : NULL);
        }
        valid &= c >= 0.0f && isfinite(c);
        response += c;
        shares[i] = c;
    }
    *coupling = shares[0] * shares[1];
    *largest = fmaxf(shares[0], shares[1]);
    return valid && isfinite(response) ? response : NAN;
}

/* block_descent_tile.cuh:743-797 InitializeTileHead */
static void init_head(tile_t *t, head_t *h, uint32_t row_index) {
    orc_env *e = t->e;
    const orc_row *row = &e->rows[row_index];
    memset(h, 0, sizeof *h);
    h->row = row_index; h->stride = row->group_normal_count;
    h->axes = (row->flags & ORC_ROW_BLOCK_NORMAL) ? 3u : 1u;
    h->flags = row->flags;
    const uint32_t owner = side_block(t, &row->a), other = side_block(t, &row->b);
    float coupling = 0.0f, largest = 0.0f;
    const float response = inertial_response(t, row, &coupling, &largest);
    const float coupled = coupling > 0.0f ? (response + sqrtf(response * response + 12.0f * coupling)) / (6.0f * coupling) : FLT_MAX;
    const float cap = 100.0f / largest;
    float rho = response > 0.0f ? fminf(cap, coupled) : 0.0f;
    if (!(response == 0.0f || (response > 0.0f && rho > 0.0f && rho <= FLT_MAX))) { e->status |= ORC_STATUS_SOLVER_FAILURE; rho = NAN; }
    h->owner[0] = owner; h->owner[1] = other == owner ? NO_BLOCK : other;
    h->rho = rho; h->compliance = row->compliance;
    h->lower = row->lower; h->upper = row->upper; h->mu1 = row->mu; h->mu2 = row->mu2;
    h->rs = float_scalar_response(rho, row->compliance);
    h->dual = V3(row->lambda, h->axes == 3u ? e->rows[row_index + h->stride].lambda : 0.0f,
                 h->axes == 3u ? e->rows[row_index + 2u * h->stride].lambda : 0.0f);
    h->base = h->dual;
}

/* block_descent_tile.cuh:659-681 TileResponse */
static void head_response(const head_t *h, v3 move, v3 *f, sym3 *c) {
    const sterm_t n = scalar_impulse(h->dual.x, h->rho, h->residual.x - move.x, h->compliance, h->lower, h->upper, h->rs);
    *f = V3(n.impulse, 0.0f, 0.0f);
    sym3 z = {n.curvature, 0, 0, 0, 0, 0};
    *c = z;
    if (h->axes != 3u) return;
    v3 ti; sym3 tc;
    tangent_impulse(h->dual, h->rho, V3(0.0f, h->residual.y - move.y, h->residual.z - move.z), h->normal_bound, h->mu1, h->mu2, &ti, &tc);
    f->y = ti.y; f->z = ti.z; c->yy = tc.yy; c->zz = tc.zz; c->yz = tc.yz;
}

static uint32_t incidence_of(const head_t *h, uint32_t block) { return h->owner[0] == block ? 0u : h->owner[1] == block ? 1u : 2u; }

/* block_descent_tile.cuh:1017-1099 IndexTileIncidence */
static void index_incidence(tile_t *t) {
    for (uint32_t b = 0; b < t->nblocks; ++b) t->blocks[b].ninc = 0;
    for (uint32_t k = 0; k < t->nheads; ++k)
        for (int s = 0; s < 2; ++s) {
            const uint32_t b = t->heads[k].owner[s];
            if (b != NO_BLOCK) t->blocks[b].inc[t->blocks[b].ninc++] = k;
        }
}

/* block_descent_tile.cuh:1103-1144 ColorTileBlocks */
static void color_blocks(tile_t *t) {
    for (uint32_t b = 0; b < t->nblocks; ++b) {
        uint32_t taken = 0u;
        for (uint32_t k = 0; k < t->blocks[b].ninc; ++k) {
            const head_t *h = &t->heads[t->blocks[b].inc[k]];
            const uint32_t other = h->owner[0] == b ? h->owner[1] : h->owner[0];
            if (other < b) taken |= 1u << t->blocks[other].color;
        }
        uint32_t c = 0; while (c < 31u && (taken >> c) & 1u) ++c;
        t->blocks[b].color = t->blocks[b].dim != 0u ? c : NO_BLOCK;
    }
}

/* block_descent_tile.cuh:891-930 InitializeTileResiduals */
static void init_residuals(tile_t *t) {
    const float dt = t->m->cfg.dt;
    for (uint32_t k = 0; k < t->nheads; ++k) {
        head_t *h = &t->heads[k];
        v3 res = V3(0, 0, 0);
        for (uint32_t ax = 0; ax < h->axes; ++ax) {
            const orc_row *row = &t->e->rows[h->row + ax * h->stride];
            float along = 0.0f;
            const orc_side *sides[2] = {&row->a, &row->b};
            for (int s = 0; s < 2; ++s) {
                float part = 0.0f;
                if (sides[s]->kind == ORC_SIDE_RIGID) {
                    const float *u = t->e->rigid_vel + 6 * sides[s]->index;
                    for (uint32_t c = 0; c < 6u; ++c) part += (c < 3u ? sides[s]->jlin[c] : sides[s]->jang[c - 3u]) * u[c];
                } else if (sides[s]->kind == ORC_SIDE_ARTIC) {
                    const float *j = s == 0 ? row->ja : row->jb;
                    if (j) for (uint32_t c = 0; c < t->blocks[t->m->B].dim; ++c) part += j[c] * t->e->artic_vel[c];
                }
                along += part;
            }
            setc3(&res, ax, row->rhs * dt - along);
        }
        h->residual = res;
    }
}

/* Cholesky H = L L^T; block_descent_tile.cuh:1623-1641 */
static int chol_factor(float *H, uint32_t n, uint32_t ld) {
    int valid = 1;
    for (uint32_t k = 0; k < n; ++k) {
        for (uint32_t i = k; i < n; ++i) {
            float v = H[i * ld + k];
            for (uint32_t j = 0; j < k; ++j) v -= H[i * ld + j] * H[k * ld + j];
            H[i * ld + k] = v;
        }
        const float pivot = H[k * ld + k];
        valid &= pivot > 0.0f && pivot <= FLT_MAX;
        const float root = sqrtf(valid ? pivot : 1.0f), scale = 1.0f / root;
        for (uint32_t i = k + 1; i < n; ++i) H[i * ld + k] *= scale;
        H[k * ld + k] = root;
    }
    return valid;
}
/* block_descent_tile.cuh:1645-1666 */
static void chol_solve(const float *Lm, uint32_t n, uint32_t ld, const float *g, float *d) {
    float r[ORC_MAX_DOF];
    for (uint32_t i = 0; i < n; ++i) r[i] = g[i];
    for (uint32_t j = 0; j < n; ++j) {
        const float y = r[j] * (1.0f / Lm[j * ld + j]);
        r[j] = y;
        for (uint32_t i = j + 1; i < n; ++i) r[i] = fmaf(-Lm[i * ld + j], y, r[i]);
    }
    for (uint32_t k = n; k > 0u; --k) {
        const uint32_t j = k - 1u;
        const float x = r[j] * (1.0f / Lm[j * ld + j]);
        r[j] = x;
        for (uint32_t i = 0; i < j; ++i) r[i] = fmaf(-Lm[j * ld + i], x, r[i]);
    }
    for (uint32_t i = 0; i < n; ++i) d[i] = r[i];
}

static int solve_block_mass(const block_t *b, const float *force, float *dir) {
    float Lm[ORC_MAX_DOF * ORC_MAX_DOF];
    const uint32_t n = b->dim;
    for (uint32_t i = 0; i < n * n; ++i) Lm[i] = b->mass[i];
    if (!chol_factor(Lm, n, n)) return 0;
    chol_solve(Lm, n, n, force, dir);
    return 1;
}

/* block_descent_tile.cuh:1508-1618 AssembleTileBlock */
static int assemble_block(tile_t *t, uint32_t bi, const float *u, const float *fr, float *H, float *force, float *inertia, int *converged) {
    const block_t *b = &t->blocks[bi];
    const uint32_t n = b->dim;
    tsum g[ORC_MAX_DOF];
    float scale[ORC_MAX_DOF], diag[ORC_MAX_DOF], diff[ORC_MAX_DOF], diff_err[ORC_MAX_DOF];
    for (uint32_t i = 0; i < n; ++i) {
        volatile float d = u[i] - fr[i];
        volatile float part = d - u[i];
        diff[i] = d; diff_err[i] = (u[i] - (d - part)) + (-fr[i] - part);
    }
    for (uint32_t i = 0; i < n; ++i) {
        tsum in = {0, 0};
        scale[i] = 0.0f; diag[i] = 0.0f;
        for (uint32_t k = 0; k < n; ++k) {
            const float mass = b->mass[i * n + k];
            H[i * n + k] = mass;
            tsum_addp(&in, mass, diff[k]);
            tsum_addp(&in, mass, diff_err[k]);
            scale[i] += fabsf(mass) * fabsf(diff[k]);
        }
        inertia[i] = in.value + in.error;
        g[i].value = -in.value; g[i].error = -in.error;
    }
    for (uint32_t k = 0; k < b->ninc; ++k) {
        const head_t *h = &t->heads[b->inc[k]];
        const uint32_t inc = incidence_of(h, bi);
        v3 f; sym3 c;
        head_response(h, h->move, &f, &c);
        const v3 noise = V3(fabsf(f.x) + c.xx * (fabsf(h->residual.x) + fabsf(h->move.x)),
                            fabsf(f.y) + c.yy * (fabsf(h->residual.y) + fabsf(h->move.y)),
                            fabsf(f.z) + c.zz * (fabsf(h->residual.z) + fabsf(h->move.z)));
        if (!(f.x != 0.0f || f.y != 0.0f || f.z != 0.0f || c.xx != 0.0f || c.yy != 0.0f || c.zz != 0.0f || c.yz != 0.0f ||
              c.xy != 0.0f || c.xz != 0.0f || noise.x != 0.0f || noise.y != 0.0f || noise.z != 0.0f)) continue;
        const float *j0 = h->jac[inc], *j1 = j0 + n, *j2 = j0 + 2 * n;
        /* a row on a single coordinate only touches that coordinate (block_descent_tile.cuh:1555-1568) */
        uint32_t supported = 0, unit = 0;
        if (h->axes == 1u) for (uint32_t i = 0; i < n; ++i) if (j0[i] != 0.0f) { ++supported; unit = i; }
        if (h->axes == 1u && supported <= 1u) {
            const float v = supported ? j0[unit] : 0.0f;
            diag[unit] += v * c.xx * v;
            tsum_addp(&g[unit], v, f.x);
            scale[unit] += fabsf(v) * noise.x;
            continue;
        }
        for (uint32_t i = 0; i < n; ++i) {
            tsum_addp(&g[i], j0[i], f.x);
            scale[i] += fabsf(j0[i]) * noise.x;
            if (h->axes == 1u) {
                const float a0 = j0[i] * c.xx;
                for (uint32_t q = 0; q < n; ++q) H[i * n + q] += a0 * j0[q];
                continue;
            }
            tsum_addp(&g[i], j1[i], f.y);
            tsum_addp(&g[i], j2[i], f.z);
            scale[i] += fabsf(j1[i]) * noise.y + fabsf(j2[i]) * noise.z;
            const float a0 = (j0[i] * c.xx + j1[i] * c.xy) + j2[i] * c.xz;
            const float a1 = (j1[i] * c.yy + j2[i] * c.yz) + j0[i] * c.xy;
            const float a2 = (j2[i] * c.zz + j1[i] * c.yz) + j0[i] * c.xz;
            for (uint32_t q = 0; q < n; ++q) H[i * n + q] += a0 * j0[q] + a1 * j1[q] + a2 * j2[q];
        }
    }
    int finite = 1, conv = 1;
    for (uint32_t i = 0; i < n; ++i) {
        H[i * n + i] += diag[i];
        force[i] = g[i].value + g[i].error;
        finite &= isfinite(force[i]);
        for (uint32_t k = 0; k < n; ++k) { finite &= isfinite(H[i * n + k]); scale[i] += fabsf(H[i * n + k]) * fabsf(u[k]); }
        conv &= fabsf(force[i]) <= ROUNDINGS * FLT_EPSILON * scale[i];
    }
    *converged = conv;
    return finite;
}

/* block_descent_tile.cuh:2019-2044 TileRowSteps */
static void row_steps(tile_t *t, uint32_t bi, const float *d) {
    const block_t *b = &t->blocks[bi];
    for (uint32_t k = 0; k < b->ninc; ++k) {
        head_t *h = &t->heads[b->inc[k]];
        const float *j = h->jac[incidence_of(h, bi)];
        v3 step = V3(0, 0, 0);
        for (uint32_t ax = 0; ax < h->axes; ++ax) {
            float s = 0.0f;
            for (uint32_t i = 0; i < b->dim; ++i) s += j[ax * b->dim + i] * d[i];
            setc3(&step, ax, s);
        }
        h->step = step;
    }
}

/* Work counters for diagnostics (single-threaded runs only): block descents, Newton steps, line evaluations. */
unsigned long long orc_work_counters[4];

/* block_descent_tile.cuh:2048-2086 TileLineDerivatives */
static void line_derivatives(tile_t *t, uint32_t bi, float alpha, float islope, float icurv, float *slope, float *curvature, float *magnitude) {
    const block_t *b = &t->blocks[bi];
    tsum rs = {0, 0};
    float rc = 0.0f, rm = 0.0f;
    ++orc_work_counters[2];
    for (uint32_t k = 0; k < b->ninc; ++k) {
        const head_t *h = &t->heads[b->inc[k]];
        const v3 trial = V3(fmaf(alpha, h->step.x, h->move.x), fmaf(alpha, h->step.y, h->move.y), fmaf(alpha, h->step.z, h->move.z));
        v3 f; sym3 c;
        head_response(h, trial, &f, &c);
        tsum_addp(&rs, f.x, h->step.x); tsum_addp(&rs, f.y, h->step.y); tsum_addp(&rs, f.z, h->step.z);
        rm += fabsf(f.x * h->step.x) + fabsf(f.y * h->step.y) + fabsf(f.z * h->step.z);
        rc += c.xx * h->step.x * h->step.x + c.yy * h->step.y * h->step.y + c.zz * h->step.z * h->step.z +
              2.0f * c.yz * h->step.y * h->step.z + 2.0f * c.xy * h->step.x * h->step.y + 2.0f * c.xz * h->step.x * h->step.z;
    }
    tsum total = {-rs.value, -rs.error};
    tsum_addp(&total, alpha, icurv);
    tsum_add(&total, islope);
    *slope = total.value + total.error;
    *curvature = icurv + rc;
    *magnitude = fabsf(islope) + alpha * icurv + rm;
}

/* block_descent_tile.cuh:2089-2125 SearchTileLine */
static float search_line(tile_t *t, uint32_t bi, float islope, float icurv) {
    float slope, curvature, magnitude;
    line_derivatives(t, bi, 0.0f, islope, icurv, &slope, &curvature, &magnitude);
    const float initial = slope;
    if (!(initial < 0.0f)) return 0.0f;
    float low = 0.0f, high = 0.0f, alpha = 1.0f;
    int bounded = 0;
    for (uint32_t step = 0; step < LINE_STEPS; ++step) {
        line_derivatives(t, bi, alpha, islope, icurv, &slope, &curvature, &magnitude);
        if (!isfinite(slope) || !isfinite(curvature)) { high = alpha; bounded = 1; alpha = 0.5f * (low + high); continue; }
        if (fabsf(slope) <= fmaxf(LINE_TOL * -initial, ROUNDINGS * FLT_EPSILON * magnitude)) return alpha;
        if (slope < 0.0f) low = alpha; else { high = alpha; bounded = 1; }
        if (bounded && high - low <= FLT_EPSILON * high) break;
        float next = alpha - slope / curvature;
        if (!(next > low && (!bounded || next < high))) next = bounded ? 0.5f * (low + high) : 2.0f * alpha;
        alpha = next;
    }
    return low;
}

static void apply_moves(tile_t *t, uint32_t bi, float alpha) {
    const block_t *b = &t->blocks[bi];
    for (uint32_t k = 0; k < b->ninc; ++k) {
        head_t *h = &t->heads[b->inc[k]];
        h->move = V3(fmaf(alpha, h->step.x, h->move.x), fmaf(alpha, h->step.y, h->move.y), fmaf(alpha, h->step.z, h->move.z));
    }
}

/* block_descent_tile.cuh:2146-2301 DescendTileBlock */
static void descend_block(tile_t *t, uint32_t bi, int position) {
    block_t *b = &t->blocks[bi];
    const uint32_t n = b->dim;
    float *velocity = position ? b->pseudo : b->vel;
    int coupled = 0;
    for (uint32_t k = 0; k < b->ninc; ++k) {       /* StartTileBlock :1386-1397 */
        head_t *h = &t->heads[b->inc[k]];
        coupled |= h->owner[0] != NO_BLOCK && h->owner[1] != NO_BLOCK;
        h->normal_bound = h->dual.x;
        h->move = V3(0, 0, 0);
    }
    float start[ORC_MAX_DOF], fr[ORC_MAX_DOF], u[ORC_MAX_DOF], d[ORC_MAX_DOF], ms[ORC_MAX_DOF];
    for (uint32_t i = 0; i < n; ++i) { start[i] = velocity[i]; fr[i] = position ? 0.0f : b->free_v[i]; u[i] = start[i]; }
    if (t->iteration == 0u && !position) {
        for (uint32_t i = 0; i < n; ++i) d[i] = fr[i] - u[i];
        tsum curv = {0, 0};
        for (uint32_t i = 0; i < n; ++i) { float s = 0.0f; for (uint32_t k = 0; k < n; ++k) s += b->mass[i * n + k] * d[k]; ms[i] = s; }
        for (uint32_t i = 0; i < n; ++i) tsum_addp(&curv, d[i], ms[i]);
        const float ic = curv.value + curv.error;
        if (ic > 0.0f && isfinite(ic)) {
            row_steps(t, bi, d);
            const float alpha = search_line(t, bi, -ic, ic);
            if (alpha > 0.0f) {
                for (uint32_t i = 0; i < n; ++i) u[i] = fmaf(alpha, d[i], u[i]);
                apply_moves(t, bi, alpha);
            }
        }
    }
    int failure = 0;
    float primal = FLT_MAX;
    ++orc_work_counters[0];
    float *H = (float *)malloc(sizeof(float) * n * n);
    for (uint32_t step = 0; step < NEWTON_STEPS; ++step) {
        float force[ORC_MAX_DOF], inertia[ORC_MAX_DOF];
        int converged = 0;
        ++orc_work_counters[1];
        /* TileNewtonDirection :1936-1992 */
        if (!assemble_block(t, bi, u, fr, H, force, inertia, &converged)) { failure = 1; break; }
        if (converged && t->tol > 0.0f) {
            if (!solve_block_mass(b, force, d)) { failure = 1; break; }
            int stationary = 1;
            for (uint32_t i = 0; i < n; ++i) stationary &= fabsf(d[i]) < t->tol;
            converged = stationary;
        }
        if (converged) { primal = 0.0f; break; }
        if (!chol_factor(H, n, n)) { failure = 1; break; }
        chol_solve(H, n, n, force, d);
        for (uint32_t i = 0; i < n; ++i) { float s = 0.0f; for (uint32_t k = 0; k < n; ++k) s += b->mass[i * n + k] * d[k]; ms[i] = s; }
        tsum dec = {0, 0}, slo = {0, 0}, cur = {0, 0};
        for (uint32_t i = 0; i < n; ++i) { tsum_addp(&dec, force[i], d[i]); tsum_addp(&slo, inertia[i], d[i]); tsum_addp(&cur, d[i], ms[i]); }
        const float total_dec = dec.value + dec.error, islope = slo.value + slo.error, icurv = cur.value + cur.error;
        if (!isfinite(total_dec) || !isfinite(islope) || !isfinite(icurv)) { failure = 1; break; }
        if (!(total_dec > 0.0f)) break;
        row_steps(t, bi, d);
        const float alpha = search_line(t, bi, islope, icurv);
        float after[ORC_MAX_DOF];
        int finite = 1, rounded = 1;
        for (uint32_t i = 0; i < n; ++i) { after[i] = fmaf(alpha, d[i], u[i]); finite &= isfinite(after[i]); rounded &= after[i] == u[i]; }
        if (!finite) { failure = 1; break; }
        primal = 0.0f;
        for (uint32_t i = 0; i < n; ++i) if (!rounded) primal = fmaxf(primal, fabsf(alpha * d[i]));
        if (!(alpha > 0.0f)) break;
        for (uint32_t i = 0; i < n; ++i) u[i] = after[i];
        apply_moves(t, bi, alpha);
        if (rounded) break;
    }
    free(H);
    for (uint32_t k = 0; k < b->ninc; ++k) {       /* EndTileBlock :1400-1409 */
        head_t *h = &t->heads[b->inc[k]];
        h->residual = V3(h->residual.x - h->move.x, h->residual.y - h->move.y, h->residual.z - h->move.z);
    }
    if (failure) t->e->status |= ORC_STATUS_SOLVER_FAILURE;
    float moved = failure ? FLT_MAX : 0.0f;
    for (uint32_t i = 0; i < n; ++i) moved = fmaxf(moved, residual_abs(u[i] - start[i]));
    t->momentum = fmaxf(t->momentum, moved);
    if (failure) primal = FLT_MAX;
    t->residual = fmaxf(t->residual, fmaxf(primal, coupled ? moved : 0.0f));
    for (uint32_t i = 0; i < n; ++i) velocity[i] = u[i];
}

/* block_descent_tile.cuh:2749-2820: colour by colour, blocks of a colour in index order */
static void descend_blocks(tile_t *t, int position) {
    for (uint32_t color = 0; color < 32u; ++color)
        for (uint32_t b = 0; b < t->nblocks; ++b)
            if (t->blocks[b].color == color) descend_block(t, b, position);
}

typedef struct { float t, beta; uint32_t restarts; } momentum_t;

/* block_descent_tile.cuh:2493-2595 UpdateTileHeadDuals */
static void update_duals(tile_t *t, momentum_t *mom, int velocity, int commit, float out[3]) {
    float cls[3] = {0, 0, 0};   /* normal, tangent, joint */
    double restart = 0.0;
    orc_env *e = t->e;
    for (uint32_t k = 0; k < t->nheads; ++k) {
        head_t *h = &t->heads[k];
        const v3 tdual = commit ? h->dual : h->base;
        const int contact = h->axes == 3u;
        const float normal = scalar_impulse(tdual.x, h->rho, h->residual.x, h->compliance, h->lower, h->upper, h->rs).impulse;
        relax_t rx = h->rx;
        if (!commit) memset(&rx, 0, sizeof rx);
        v3 dual;
        if (!contact) dual = V3(normal, 0, 0);
        else {
            v3 ti; sym3 tc;
            tangent_impulse(tdual, h->rho, h->residual, normal, h->mu1, h->mu2, &ti, &tc);
            dual = relax_contact_impulse(tdual, V3(normal, ti.y, ti.z), &rx);
        }
        float sn, st;
        multiplier_steps(tdual, dual, h->rs.residual_scale, h->rs.dual_scale, h->rho, contact ? h->mu1 : 0.0f, contact ? h->mu2 : 0.0f, &sn, &st);
        if (!commit && h->rs.residual_scale > 0.0f) sn = fabsf(dual.x - tdual.x) / h->rs.residual_scale;
        const v3 physical = commit ? dual : tdual;
        if (!contact) {
            const int normal_row = (h->flags & ORC_ROW_CONTACT_NORMAL) != 0u;
            const float rate = -h->residual.x + h->compliance * physical.x;
            const float violation = physical.x > 0.0f ? fabsf(rate) : fmaxf(-rate, 0.0f);
            const float r = normal_row ? fmaxf(sn, violation) : sn;
            float *c = normal_row ? &cls[0] : &cls[2];
            *c = fmaxf(*c, residual_abs(r));
        } else {
            if (commit) {
                h->rx = rx;
                e->rows[h->row + h->stride].lambda = dual.y;
                e->rows[h->row + 2u * h->stride].lambda = dual.z;
            }
            const v3 v = V3(-h->residual.x + h->compliance * physical.x, -h->residual.y, -h->residual.z);
            cls[0] = fmaxf(cls[0], residual_abs(physical.x > 0.0f ? fabsf(v.x) : fmaxf(-v.x, 0.0f)));
            cls[1] = fmaxf(cls[1], residual_abs(fmaxf(st, fmaxf(along_axis(physical.y, v.y), along_axis(physical.z, v.z)))));
        }
        if (!commit) continue;
        if (velocity) e->rows[h->row].lambda = dual.x;
        const int extrapolate = contact || h->rs.dual_scale != 0.0f;
        const v3 metric = multiplier_metric(h->rs.residual_scale, h->rho, contact, h->mu1, h->mu2);
        if (extrapolate) restart += momentum_restart(tdual, dual, h->base, metric);
        if (mom) h->move = h->base;
        h->dual = dual;
        h->base = dual;
    }
    if (mom) {
        /* block_descent.cu:780-788 AdvanceDualMomentum */
        if (restart > 0.0) { mom->t = 1.0f; ++mom->restarts; }
        const float tn = 0.5f * (1.0f + sqrtf(fmaf(4.0f * mom->t, mom->t, 1.0f)));
        mom->beta = (mom->t - 1.0f) / tn;
        mom->t = tn;
        for (uint32_t k = 0; k < t->nheads; ++k) {
            head_t *h = &t->heads[k];
            const int contact = h->axes == 3u;
            const int extrapolate = contact || h->rs.dual_scale != 0.0f;
            h->dual = extrapolate_dual(h->move, h->base, extrapolate ? mom->beta : 0.0f, h->lower, h->upper, contact, h->mu1, h->mu2);
        }
    }
    out[0] = cls[0]; out[1] = cls[1]; out[2] = cls[2];
}

/* block_descent_tile.cuh:2379-2489 MeasureTilePrimal over every moving block */
static void measure_primals(tile_t *t, int reconstruct) {
    orc_env *e = t->e;
    for (uint32_t color = 0; color < 32u; ++color) for (uint32_t bi = 0; bi < t->nblocks; ++bi) {
        block_t *b = &t->blocks[bi];
        if (b->color != color) continue;
        const uint32_t n = b->dim;
        double balance[ORC_MAX_DOF];
        for (uint32_t i = 0; i < n; ++i) {
            balance[i] = 0.0;
            for (uint32_t j = 0; j < n; ++j) balance[i] -= (double)b->mass[i * n + j] * ((double)b->vel[j] - b->free_v[j]);
        }
        for (uint32_t k = 0; k < b->ninc; ++k) {
            const head_t *h = &t->heads[b->inc[k]];
            const float *jac = h->jac[incidence_of(h, bi)];
            for (uint32_t ax = 0; ax < h->axes; ++ax) {
                const float imp = e->rows[h->row + ax * h->stride].lambda;
                if (imp == 0.0f) continue;
                for (uint32_t i = 0; i < n; ++i) balance[i] += (double)jac[ax * n + i] * imp;
            }
        }
        float force[ORC_MAX_DOF], dir[ORC_MAX_DOF];
        int finite = 1;
        for (uint32_t i = 0; i < n; ++i) { force[i] = (float)balance[i]; finite &= fabs(balance[i]) <= FLT_MAX; }
        int ok = finite && solve_block_mass(b, force, dir);
        float residual = ok ? 0.0f : FLT_MAX;
        if (ok) for (uint32_t i = 0; i < n; ++i) residual = fmaxf(residual, isfinite(dir[i]) ? fabsf(dir[i]) : FLT_MAX);
        t->residual = fmaxf(t->residual, residual);
        if (reconstruct && ok) {
            for (uint32_t i = 0; i < n; ++i) b->vel[i] += dir[i];
            t->momentum = fmaxf(t->momentum, residual);
        }
    }
}

/* block_descent.cu:1734-1753 PositionRowBias */
static void position_row_bias(const tile_t *t, const orc_row *row, float slop, float *bias, float *rounding) {
    const orc_config *cfg = &t->m->cfg;
    const orc_env *e = t->e;
    const float penetration = fmaxf(row->penetration - slop, 0.0f);
    if ((row->flags & ORC_ROW_SPECULATIVE) != 0u) {
        const uint32_t pt = row->contact_slot * 4u + row->contact_point;
        const double depth = (double)e->cdepth[pt] - slop;
        const double reserve = (double)row->penetration - e->cdepth[pt];
        const double correction = cfg->pos_beta * fmax(depth, 0.0) + reserve;
        const double target = fmin(depth, 0.0) + correction;
        double velocity = 0.0;        /* RowVelocity :1051-1082 on the solved velocities */
        const orc_side *sides[2] = {&row->a, &row->b};
        for (int s = 0; s < 2; ++s) {
            if (sides[s]->kind == ORC_SIDE_RIGID) {
                const float *lv = e->body_linvel + 3 * sides[s]->index, *av = e->body_angvel + 3 * sides[s]->index;
                velocity += (double)sides[s]->jlin[0] * lv[0] + (double)sides[s]->jlin[1] * lv[1] + (double)sides[s]->jlin[2] * lv[2] +
                            (double)sides[s]->jang[0] * av[0] + (double)sides[s]->jang[1] * av[1] + (double)sides[s]->jang[2] * av[2];
            } else if (sides[s]->kind == ORC_SIDE_ARTIC) {
                const float *j = s == 0 ? row->ja : row->jb;
                double v = 0.0;
                if (j) for (uint32_t d = 0; d < t->m->ndof; ++d) v += (double)j[d] * e->artic_vel[d];
                velocity += v;
            }
        }
        const double limit = fmin(correction / cfg->dt, (double)cfg->baumgarte_max_velocity);
        const double absorbed = target > 0.0 ? 0.0 : fmax(reserve, 0.0) / cfg->dt;
        *bias = (float)fmin(target / cfg->dt - velocity, limit);
        *rounding = (float)absorbed;
        return;
    }
    const float correction = cfg->pos_beta * penetration + fmaxf(penetration - penetration, 0.0f);
    *bias = fminf(correction / cfg->dt, cfg->baumgarte_max_velocity);
    *rounding = 0.0f;
}

/* rigid block setup, block_descent_rigid.cuh:4-48 */
static void init_rigid_block(tile_t *t, uint32_t body, block_t *b) {
    const orc_model *m = t->m; orc_env *e = t->e;
    float *fr = e->rigid_free + 6 * body;
    memcpy(fr, e->body_linvel + 3 * body, 12); memcpy(fr + 3, e->body_angvel + 3 * body, 12);
    b->dim = 0;
    const float im = m->inv_mass[body];
    if (im == 0.0f) return;
    const float *w = e->body_winv + 6 * body;
    const double xx = w[0], yy = w[1], zz = w[2], xy = w[3], xz = w[4], yz = w[5];
    const double cxx = yy * zz - yz * yz, cyy = xx * zz - xz * xz, czz = xx * yy - xy * xy;
    const double cxy = xz * yz - xy * zz, cxz = xy * yz - xz * yy, cyz = xy * xz - xx * yz;
    const double det = xx * cxx + xy * cxy + xz * cxz;
    if (!(im > 0.0f) || !(det > 0.0)) { e->status |= ORC_STATUS_SOLVER_FAILURE; return; }
    const double inv = 1.0 / det;
    const float I[6] = {(float)(cxx * inv), (float)(cyy * inv), (float)(czz * inv), (float)(cxy * inv), (float)(cxz * inv), (float)(cyz * inv)};
    const float rot[3][3] = {{I[0], I[3], I[4]}, {I[3], I[1], I[5]}, {I[4], I[5], I[2]}};
    const float mass = (float)(1.0 / (double)im);
    for (uint32_t r = 0; r < 6u; ++r) for (uint32_t c = 0; c < 6u; ++c) {
        float v = 0.0f;
        if (r < 3u && c < 3u && r == c) v = mass;
        if (r >= 3u && c >= 3u) v = rot[r - 3u][c - 3u];
        b->mass[r * 6u + c] = v;
    }
    b->dim = 6u;
}

/* ops/block_descent_tile.cuh:2942-3087 DescendTile */
void orc_solve(const orc_model *m, orc_env *e) {
    tile_t t; memset(&t, 0, sizeof t);
    t.m = m; t.e = e; t.tol = m->cfg.velocity_tolerance;
    const uint32_t nb = m->B + (m->L > 0u ? 1u : 0u);
    t.nblocks = nb;
    t.blocks = (block_t *)calloc(nb ? nb : 1u, sizeof(block_t));
    float *rigid_mass = (float *)calloc((size_t)m->B * 36u + 1u, sizeof(float));
    uint32_t *inc_pool = (uint32_t *)calloc((size_t)nb * (e->nrows + 1u), sizeof(uint32_t));
    /* InitializeTile :1301-1357: blocks start from their free velocity plus the carried constraint velocity */
    for (uint32_t b = 0; b < m->B; ++b) {
        block_t *bl = &t.blocks[b];
        bl->mass = rigid_mass + 36u * b; bl->inc = inc_pool + (size_t)b * (e->nrows + 1u);
        bl->free_v = e->rigid_free + 6 * b; bl->vel = e->rigid_vel + 6 * b; bl->pseudo = e->body_pseudo + 6 * b;
        float carried[6];
        for (int i = 0; i < 6; ++i) carried[i] = bl->vel[i] - bl->free_v[i];
        init_rigid_block(&t, b, bl);
        for (int i = 0; i < 6; ++i) bl->vel[i] = bl->free_v[i] + (isfinite(carried[i]) ? carried[i] : 0.0f);
    }
    if (m->L > 0u) {
        block_t *bl = &t.blocks[m->B];
        bl->dim = m->ndof; bl->mass = e->M; bl->inc = inc_pool + (size_t)m->B * (e->nrows + 1u);
        bl->free_v = e->artic_free; bl->vel = e->artic_vel; bl->pseudo = e->qdot_pseudo;
        uint32_t d = 0;
        for (uint32_t l = 0; l < m->L; ++l) {
            const uint32_t t_ = m->jtype[l];
            const uint32_t w = (t_ == ORC_JOINT_REVOLUTE || t_ == ORC_JOINT_PRISMATIC) ? 1u : t_ == ORC_JOINT_FLOATING ? 6u : 0u;
            for (uint32_t c = 0; c < w; ++c, ++d) {
                const float value = w == 1u ? e->qdot[l] : e->link_vel[6 * l + c];
                const float carried = e->artic_vel[d] - e->artic_free[d];
                e->artic_free[d] = value;
                e->artic_vel[d] = value + (isfinite(carried) ? carried : 0.0f);
            }
        }
    }
    /* heads in row order :1257-1296 */
    t.heads = (head_t *)calloc(e->nrows + 1u, sizeof(head_t));
    for (uint32_t r = 0; r < e->nrows; ++r) {
        const uint32_t fl = e->rows[r].flags;
        if ((fl & ORC_ROW_ACTIVE) && !(fl & ORC_ROW_BLOCK_TANGENT)) init_head(&t, &t.heads[t.nheads++], r);
    }
    index_incidence(&t);
    color_blocks(&t);
    /* staged Jacobians :837-869 */
    size_t jac_floats = 0;
    for (uint32_t k = 0; k < t.nheads; ++k) for (int s = 0; s < 2; ++s)
        if (t.heads[k].owner[s] != NO_BLOCK) jac_floats += (size_t)t.heads[k].axes * t.blocks[t.heads[k].owner[s]].dim;
    float *jac_pool = (float *)calloc(jac_floats + 1u, sizeof(float)), *jp = jac_pool;
    for (uint32_t k = 0; k < t.nheads; ++k) for (int s = 0; s < 2; ++s) {
        head_t *h = &t.heads[k];
        const uint32_t b = h->owner[s];
        if (b == NO_BLOCK) continue;
        h->jac[s] = jp;
        for (uint32_t ax = 0; ax < h->axes; ++ax) for (uint32_t i = 0; i < t.blocks[b].dim; ++i)
            *jp++ = block_jacobian(&t, b, &e->rows[h->row + ax * h->stride], i);
    }
    init_residuals(&t);
    float rows[3] = {0, 0, 0}, residual_cls[4] = {0, 0, 0, 0};
    uint32_t sweeps = 0;
    momentum_t mom = {1.0f, 0.0f, 0u};
    const uint32_t iterations = m->cfg.vel_iters;
    while (sweeps < iterations) {
        t.iteration = sweeps++;
        t.momentum = 0.0f; t.residual = 0.0f;
        descend_blocks(&t, 0);
        update_duals(&t, &mom, 1, 1, rows);
        if (sweeps == iterations || fmaxf(fmaxf(rows[0], rows[1]), fmaxf(rows[2], t.residual)) < t.tol) measure_primals(&t, 0);
        if (fmaxf(fmaxf(rows[0], rows[1]), rows[2]) < t.tol && t.residual >= t.tol && t.residual < FLT_MAX) {
            measure_primals(&t, 1);
            if (t.residual < FLT_MAX) {
                init_residuals(&t);
                update_duals(&t, NULL, 1, 0, rows);
                t.residual = 0.0f;
                measure_primals(&t, 0);
            }
        }
        residual_cls[0] = rows[0]; residual_cls[1] = rows[1]; residual_cls[2] = rows[2]; residual_cls[3] = t.residual;
        const float largest = fmaxf(fmaxf(rows[0], rows[1]), fmaxf(rows[2], t.residual));
        if (largest < t.tol || largest == FLT_MAX) break;
    }
    memcpy(e->solver_residual, residual_cls, sizeof residual_cls);
    e->sweeps = sweeps;
    /* FinishTile :2608-2669 */
    if (m->L > 0u) {
        uint32_t d = 0;
        for (uint32_t l = 0; l < m->L; ++l) {
            const uint32_t t_ = m->jtype[l];
            const uint32_t w = (t_ == ORC_JOINT_REVOLUTE || t_ == ORC_JOINT_PRISMATIC) ? 1u : t_ == ORC_JOINT_FLOATING ? 6u : 0u;
            for (uint32_t c = 0; c < w; ++c, ++d) { if (w == 1u) e->qdot[l] = e->artic_vel[d]; else e->link_vel[6 * l + c] = e->artic_vel[d]; }
        }
    }
    for (uint32_t b = 0; b < m->B; ++b) {
        if (t.blocks[b].dim == 0u) continue;
        memcpy(e->body_linvel + 3 * b, e->rigid_vel + 6 * b, 12);
        memcpy(e->body_angvel + 3 * b, e->rigid_vel + 6 * b + 3, 12);
    }
    /* split-impulse position pass :2673-2717, 3059-3077 */
    for (uint32_t d = 0; d < m->ndof; ++d) e->qdot_pseudo[d] = 0.0f;
    for (uint32_t k = 0; k < m->B * 6u; ++k) e->body_pseudo[k] = 0.0f;
    if (m->cfg.pos_iters != 0u && e->row_cap > 0u) {
        int push = 0, coupled = 0;
        for (uint32_t k = 0; k < t.nheads; ++k) {
            head_t *h = &t.heads[k];
            const orc_row *row = &e->rows[h->row];
            const float slop = (row->flags & ORC_ROW_SPECULATIVE) ? 0.0f : m->cfg.pos_slop;
            const int position = (row->flags & ORC_ROW_VELOCITY_ONLY) == 0u &&
                ((row->flags & ORC_ROW_SPECULATIVE) != 0u || row->penetration > slop || h->dual.x != 0.0f);
            float bias = 0.0f, rounding = 0.0f;
            if (position) position_row_bias(&t, row, slop, &bias, &rounding);
            if (!position) h->owner[0] = h->owner[1] = NO_BLOCK;
            coupled |= h->owner[0] != NO_BLOCK && h->owner[1] != NO_BLOCK;
            h->axes = 1u; h->compliance = 0.0f; h->lower = 0.0f; h->upper = FLT_MAX;
            h->rs = float_scalar_response(h->rho, 0.0f);
            h->residual = V3(bias, 0, 0);
            h->dual = V3(0, 0, 0);
            push |= bias > rounding;
        }
        if (push) {
            index_incidence(&t);
            const uint32_t positions = coupled ? m->cfg.pos_iters : 1u;
            for (uint32_t it = 0; it < positions; ++it) {
                t.iteration = sweeps + it;
                descend_blocks(&t, 1);
                if (it + 1u < positions) update_duals(&t, NULL, 0, 1, rows);
            }
        }
    }
    free(jac_pool); free(t.heads); free(inc_pool); free(rigid_mass); free(t.blocks);
}


/* Known-answer access for tests: the row laws of nk/solve/augmented_row.hpp.
 * which 0: momentum_restart(point, next, base, scale) -> out[0] (in: 12 floats)
 * which 1: two relaxation steps of tests/math/test_contact_tangent.cpp:20-35 (in[0] = beta) -> root xyz, weight
 * which 2: tangent_impulse(dual 0, rho in[0], residual in[1..3], normal in[4], mu in[5] both axes) -> iy, iz, yy, zz, yz */
void orc_law_kat(int which, const float *in, double *out) {
    if (which == 0) {
        out[0] = momentum_restart(V3(in[0], in[1], in[2]), V3(in[3], in[4], in[5]), V3(in[6], in[7], in[8]), V3(in[9], in[10], in[11]));
    } else if (which == 1) {
        relax_t history;
        memset(&history, 0, sizeof history);
        const v3 start = V3(10.0f, 1.0f, 0.0f);
        const v3 first = relax_contact_impulse(start, V3(10.0f, -2.0f, 0.0f), &history);
        const v3 point = V3(first.x + (first.x - start.x) * in[0], first.y + (first.y - start.y) * in[0], first.z + (first.z - start.z) * in[0]);
        const v3 root = relax_contact_impulse(point, V3(10.0f, -2.0f * point.y, 0.0f), &history);
        out[0] = root.x; out[1] = root.y; out[2] = root.z; out[3] = history.weight;
    } else if (which == 2) {
        v3 impulse = V3(0, 0, 0);
        sym3 curv;
        memset(&curv, 0, sizeof curv);
        tangent_impulse(V3(0, 0, 0), in[0], V3(in[1], in[2], in[3]), in[4], in[5], in[5], &impulse, &curv);
        out[0] = impulse.y; out[1] = impulse.z; out[2] = curv.yy; out[3] = curv.zz; out[4] = curv.yz;
    }
}

/* Differential-test access: the row laws over n records, same record layouts as the reference-header binding
 * (oracle/ref_headers.cpp: ref_law_batch), which 0..4. */
void orc_law_batch(int which, uint32_t n, const float *in, uint32_t in_stride, float *out, uint32_t out_stride) {
    for (uint32_t i = 0; i < n; ++i) {
        const float *x = in + (size_t)i * in_stride;
        float *o = out + (size_t)i * out_stride;
        if (which == 0) {
            const sterm_t t = scalar_impulse(x[0], x[1], x[2], x[3], x[4], x[5], float_scalar_response(x[1], x[3]));
            o[0] = t.impulse; o[1] = t.curvature;
        } else if (which == 1) {
            o[0] = cone_argument(x[0], x[1], x[2], x[3]);
        } else if (which == 2) {
            v3 impulse; sym3 curv;
            tangent_impulse(V3(0.0f, x[0], x[1]), x[2], V3(0.0f, x[3], x[4]), x[5], x[6], x[7], &impulse, &curv);
            o[0] = impulse.y; o[1] = impulse.z; o[2] = curv.yy; o[3] = curv.zz; o[4] = curv.yz;
        } else if (which == 3) {
            o[0] = (float)momentum_restart(V3(x[0], x[1], x[2]), V3(x[3], x[4], x[5]), V3(x[6], x[7], x[8]), V3(x[9], x[10], x[11]));
        } else if (which == 4) {
            relax_t last = {V3(x[6], x[7], x[8]), x[9], V3(x[10], x[11], x[12])};
            const v3 r = relax_contact_impulse(V3(x[0], x[1], x[2]), V3(x[3], x[4], x[5]), &last);
            o[0] = r.x; o[1] = r.y; o[2] = r.z; o[3] = last.weight;
        }
    }
}
