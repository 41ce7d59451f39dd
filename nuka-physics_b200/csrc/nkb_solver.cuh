// Warp-per-env block-descent velocity solve with split-impulse position pass.
// Blocks are the env's free bodies (6 coordinates: linear, angular) followed by its articulation (one
// coordinate per DoF).  Blocks descend colour by colour; each block takes safeguarded Newton steps with an
// exact line search on its local augmented Lagrangian, then the multipliers update with momentum.
// One lane owns one block coordinate in the Newton system and one head in the row evaluations.
// The algorithm is that of the reference's tile route: ops/block_descent_tile.cuh:743-797 (head setup),
// :1103-1144 (colouring), :1508-1666 (assemble/factor/solve), :2089-2301 (line search, block descent),
// :2493-2595 (dual update), :2379-2489 (momentum balance), :2608-2744 (finish, position marks),
// :2942-3087 (sweep loop) and ops/block_descent.cu:1734-1753 (position bias).
#pragma once
#include "nkb_laws.cuh"
#include "nkb_rows.cuh"

namespace nkb {

static_assert(HF_COUNT == kHeadWords, "head field count must match the host layout");

constexpr uint32_t kNewtonSteps = 16u, kLineSteps = 32u;
constexpr float kLineTol = 1.0e-6f, kRoundings = 8.0f;

struct Tile {
    uint32_t nheads, nblocks, iteration;
    float momentum, residual, tol;
};

NKB_DEV uint32_t* sm_binfo(const Env& e) { return reinterpret_cast<uint32_t*>(e.sm + e.lay->binfo); }
// binfo words: dim[nb], color[nb], inc_begin[nb + 1], inc[2 * head_cap], utab[4 * vstride], order[nb + 1]
NKB_DEV uint32_t& blk_dim(const Env& e, uint32_t b) { return sm_binfo(e)[b]; }
NKB_DEV uint32_t& blk_color(const Env& e, uint32_t nb, uint32_t b) { return sm_binfo(e)[nb + b]; }
NKB_DEV uint32_t& blk_inc_begin(const Env& e, uint32_t nb, uint32_t b) { return sm_binfo(e)[2u * nb + b]; }
NKB_DEV uint32_t* blk_inc(const Env& e, uint32_t nb) { return sm_binfo(e) + 3u * nb + 1u; }
// unit rows of the articulation by coordinate: utab[slot * vstride + coordinate] = head or 0xffff (slots: lower limit,
// upper limit, dry friction, drive; vstride = 32 or 64 coordinates), 16-bit entries
constexpr uint32_t kNoUnitHead = 0xffffu;
NKB_DEV uint16_t* unit_table(const Env& e, uint32_t nb) { return reinterpret_cast<uint16_t*>(sm_binfo(e) + 3u * nb + 1u + 2u * e.t->head_cap); }
// moving blocks in descent order, order[nb] = their count
NKB_DEV uint32_t* block_order(const Env& e, uint32_t nb) { return sm_binfo(e) + 3u * nb + 1u + 2u * e.t->head_cap + 2u * e.vstride; }
NKB_DEV float* sm_bmass(const Env& e, uint32_t b) { return e.sm + e.lay->bmass + 7u * free_slot(e, b); }
NKB_DEV float* sm_bfree(const Env& e, uint32_t b) { return e.sm + e.lay->bfree + 6u * free_slot(e, b); }
NKB_DEV float* sm_bpseudo(const Env& e, uint32_t b) { return e.sm + e.lay->bpseudo + 6u * free_slot(e, b); }

NKB_DEV uint32_t head_axes(const Env& e, uint32_t h) { return (hu(e, HF_FLAGS, h) & (kHeadContact | kHeadScalar)) == kHeadContact ? 3u : 1u; }
NKB_DEV uint32_t head_owner(const Env& e, uint32_t h, uint32_t side) { const uint32_t o = hu(e, HF_OWNER, h); return side == 0u ? (o & 0xffffu) : (o >> 16); }

// Jacobian entry of head h (incidence `side`) on coordinate i of its block, for contact axis ax.
NKB_DEV float head_jac(const Env& e, uint32_t h, uint32_t side, uint32_t ax, uint32_t i, uint32_t block) {
    const TemplateView& t = *e.t;
    if (block == t.B) {
        const uint32_t jo = hu(e, HF_JOFF, h);
        if (jo & kUnitRow) return i == (jo & 0xffffu) ? hf(e, HF_UNITV, h) : 0.f;
        return sm_jpool(e)[jo + ax * ((t.ndof + 3u) & ~3u) + i];
    }
    const V3 dir = hf3(e, ax == 0u ? HF_N : ax == 1u ? HF_T1 : HF_T2, h);
    const float sgn = side == 0u ? 1.f : -1.f;
    if (i < 3u) return sgn * comp(dir, (int)i);
    const V3 r = hf3(e, side == 0u ? HF_RA : HF_RB, h);
    return sgn * comp(cross(r, dir), (int)i - 3);
}

// J_h[ax] . u over the coordinates of block b (u padded with zeros to a multiple of 4 for the articulation).
NKB_DEV float head_row_dot(const Env& e, uint32_t h, uint32_t side, uint32_t ax, uint32_t block, const float* u) {
    const TemplateView& t = *e.t;
    if (block == t.B) {
        const uint32_t jo = hu(e, HF_JOFF, h);
        if (jo & kUnitRow) return hf(e, HF_UNITV, h) * u[jo & 0xffffu];
        const uint32_t chunks = (t.ndof + 3u) >> 2;
        const float4* j4 = reinterpret_cast<const float4*>(sm_jpool(e) + jo) + ax * chunks;
        const float4* u4 = reinterpret_cast<const float4*>(u);
        float s = 0.f;
#pragma unroll 1
        for (uint32_t c = 0u; c < chunks; ++c) {
            const float4 a = j4[c], b4 = u4[c];
            s = fmaf(a.x, b4.x, s); s = fmaf(a.y, b4.y, s); s = fmaf(a.z, b4.z, s); s = fmaf(a.w, b4.w, s);
        }
        return s;
    }
    float s = 0.f;
#pragma unroll 1
    for (uint32_t i = 0u; i < 6u; ++i) s += head_jac(e, h, side, ax, i, block) * u[i];
    return s;
}

// Mass entry (i, k) of a block.
NKB_DEV float block_mass(const Env& e, uint32_t block, uint32_t i, uint32_t k) {
    if (block == e.t->B) return sm_mass(e)[i * e.lay->ld + k];
    const float* bm = sm_bmass(e, block);
    if (i < 3u || k < 3u) return (i == k) ? bm[0] : 0.f;
    const uint32_t a = i - 3u, b = k - 3u;
    const uint32_t idx = a == b ? a : (a + b == 1u ? 3u : a + b == 2u ? 4u : 5u);
    return bm[1u + idx];
}
NKB_DEV float* block_vel(const Env& e, uint32_t block, bool position) {
    if (block == e.t->B) return sm_vec(e, position ? kVecPseudo : kVecU);
    return position ? sm_bpseudo(e, block) : sm_bvel(e, block);
}
NKB_DEV const float* block_free(const Env& e, uint32_t block) { return block == e.t->B ? sm_vec(e, kVecFree) : sm_bfree(e, block); }

// x = M^-1 g for a block; a lane holds coordinates lane + 32 r.
template <int NR>
NKB_DEV void solve_block_mass(const Env& e, uint32_t block, const float (&g)[NR], float (&x)[NR]) {
    const TemplateView& t = *e.t;
    const uint32_t l = e.lane;
    if (block == t.B) {
        const uint32_t n = t.ndof, ld = e.lay->ld;
        const float* F = sm_factor(e);
#pragma unroll
        for (int r = 0; r < NR; ++r) x[r] = l + 32u * r < n ? g[r] : 0.f;
#pragma unroll 1
        for (uint32_t j = 0; j < n; ++j) {
            const float xj = coord_bcast<NR>(x, j);
#pragma unroll
            for (int r = 0; r < NR; ++r) { const uint32_t row = l + 32u * r; if (row > j && row < n) x[r] -= F[row * ld + j] * xj; }
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) { const uint32_t row = l + 32u * r; if (row < n) x[r] /= F[row * ld + row]; }
#pragma unroll 1
        for (uint32_t jj = n; jj > 0u; --jj) {
            const uint32_t j = jj - 1u;
            const float xj = coord_bcast<NR>(x, j);
#pragma unroll
            for (int r = 0; r < NR; ++r) { const uint32_t row = l + 32u * r; if (row < j) x[r] -= F[j * ld + row] * xj; }
        }
        return;
    }
    const float g3 = __shfl_sync(NKB_FULL, g[0], 3), g4 = __shfl_sync(NKB_FULL, g[0], 4), g5 = __shfl_sync(NKB_FULL, g[0], 5);
#pragma unroll
    for (int r = 0; r < NR; ++r) x[r] = 0.f;
    if (l < 3u) x[0] = g[0] * __ldg(t.inv_mass + block);
    else if (l < 6u) { const V3 w = sym_mulv(sm_bwinv(e, block), mk3(g3, g4, g5)); x[0] = comp(w, (int)l - 3); }
}

// J M^-1 J^T of an articulated row from one forward solve with the unit-lower factor (articulation_mass.cuh:413-441)
// Row with a single entry `value` at coordinate `at`: the solve starts there, the leading zeros contribute nothing.
template <int NR>
NKB_DEV float mass_coupling_unit(const Env& e, uint32_t at, float value) {
    const uint32_t n = e.t->ndof, ld = e.lay->ld;
    const float* F = sm_factor(e);
    float y[32 * NR];
    float r = 0.f;
    for (uint32_t i = at; i < n; ++i) {
        float a = i == at ? value : 0.f;
        for (uint32_t j = at; j < i; ++j) a -= F[i * ld + j] * y[j];
        y[i] = a;
        r += a * a / F[i * ld + i];
    }
    return r;
}

// The same for dense rows (contact rows against the articulation), all lanes on one row at a time: lane = coordinate
// in the forward solve, then lane = row adds its row's terms in coordinate order, so the sum is the sequential one.
// Results land in HF_RSD of each head (a field init_heads fills afterwards).
template <int NR>
NKB_DEV void mass_coupling_dense(Env& e, const Tile& tile) {
    const TemplateView& t = *e.t;
    const uint32_t n = t.ndof, ld = e.lay->ld, l = e.lane;
    if (n == 0u) return;
    const float* F = sm_factor(e);
    float* terms = e.sm + e.lay->chol;                  // Newton scratch, free until the first descent: >= n x n words
    const uint32_t batch = n < 32u ? n : 32u;           // rows per batch
    float diag[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) { const uint32_t c = l + 32u * r; diag[r] = c < n ? F[c * ld + c] : 1.f; }
    for (uint32_t base = 0u; base < tile.nheads; base += 32u) {
        const uint32_t h = base + l;
        bool dense = false;
        if (h < tile.nheads) {
            const uint32_t o = hu(e, HF_OWNER, h);
            dense = ((o & 0xffffu) == t.B || (o >> 16) == t.B) && !(hu(e, HF_JOFF, h) & kUnitRow);
        }
        uint32_t todo = __ballot_sync(NKB_FULL, dense);
        while (todo != 0u) {
            uint32_t in_batch = 0u, mine = 0xffffffffu;
#pragma unroll 1
            for (; todo != 0u && in_batch < batch; ++in_batch) {
                const uint32_t src = (uint32_t)__ffs(todo) - 1u;
                todo &= todo - 1u;
                if (l == src) mine = in_batch;
                const float* row = sm_jpool(e) + hu(e, HF_JOFF, base + src);
                float x[NR];
#pragma unroll
                for (int r = 0; r < NR; ++r) { const uint32_t c = l + 32u * r; x[r] = c < n ? row[c] : 0.f; }
#pragma unroll 1
                for (uint32_t j = 0u; j < n; ++j) {
                    const float xj = coord_bcast<NR>(x, j);
#pragma unroll
                    for (int r = 0; r < NR; ++r) { const uint32_t c = l + 32u * r; if (c > j && c < n) x[r] -= F[c * ld + j] * xj; }
                }
#pragma unroll
                for (int r = 0; r < NR; ++r) { const uint32_t c = l + 32u * r; if (c < n) terms[in_batch * n + c] = x[r] * x[r] / diag[r]; }
            }
            __syncwarp();
            if (mine != 0xffffffffu) {
                float r = 0.f;
                for (uint32_t i = 0u; i < n; ++i) r += terms[mine * n + i];
                hf(e, HF_RSD, h) = r;
            }
            __syncwarp();
        }
    }
}

// Head setup: penalty, response scales (block_descent_tile.cuh:743-797).
template <int NR>
NKB_DEV void init_heads(Env& e, const Tile& tile) {
    const TemplateView& t = *e.t;
    mass_coupling_dense<NR>(e, tile);
    for (uint32_t h = e.lane; h < tile.nheads; h += 32u) {
        float shares[2] = {0.f, 0.f};
        const uint32_t fl = hu(e, HF_FLAGS, h);
        const uint32_t jo = hu(e, HF_JOFF, h);
        bool valid = true;
        for (uint32_t side = 0u; side < 2u; ++side) {
            const uint32_t ob = head_owner(e, h, side);
            float c = 0.f;
            if (ob == kNoBlock16) { /* static or kinematic side: no response */ }
            else if (ob == t.B) {
                if (jo & kUnitRow) c = mass_coupling_unit<NR>(e, jo & 0xffffu, hf(e, HF_UNITV, h));
                else c = hf(e, HF_RSD, h);
            } else {
                const V3 dir = hf3(e, HF_N, h) * (side == 0u ? 1.f : -1.f);
                const V3 ang = cross(hf3(e, side == 0u ? HF_RA : HF_RB, h), dir);
                c = __ldg(t.inv_mass + ob) * dot(dir, dir) + dot(ang, sym_mulv(sm_bwinv(e, ob), ang));
            }
            valid &= c >= 0.f && isfinite(c);
            shares[side] = c;
        }
        const float response = (valid && isfinite(shares[0] + shares[1])) ? shares[0] + shares[1] : nanf("");
        const float coupling = shares[0] * shares[1], largest = fmaxf(shares[0], shares[1]);
        const float coupled = coupling > 0.f ? (response + sqrtf(response * response + 12.0f * coupling)) / (6.0f * coupling) : FLT_MAX;
        const float cap = 100.0f / largest;
        float rho = response > 0.f ? fminf(cap, coupled) : 0.f;
        if (!(response == 0.f || (response > 0.f && rho > 0.f && rho <= FLT_MAX))) { e.status |= kStatusSolverFailure; rho = nanf(""); }
        const Resp rs = scalar_response(rho, 0.0f);
        hf(e, HF_RHO, h) = rho; hf(e, HF_RSD, h) = rs.dual_scale; hf(e, HF_RSR, h) = rs.residual_scale;
        hf(e, HF_NB, h) = 0.f;
        hst3(e, HF_BASE, h, hf3(e, HF_DUAL, h));
        hst3(e, HF_RES, h, mk3(0.f, 0.f, 0.f)); hst3(e, HF_MOVE, h, mk3(0.f, 0.f, 0.f)); hst3(e, HF_STEP, h, mk3(0.f, 0.f, 0.f));
        hst3(e, HF_RXS, h, mk3(0.f, 0.f, 0.f)); hf(e, HF_RXW, h) = 0.f; hst3(e, HF_RXP, h, mk3(0.f, 0.f, 0.f));
        (void)fl;
    }
    __syncwarp();
}

// Incidence lists (heads of each block in head order) and greedy colours.
NKB_DEV void index_blocks(Env& e, const Tile& tile, bool color) {
    const uint32_t nb = tile.nblocks;
    uint32_t* inc = blk_inc(e, nb);
    uint32_t at = 0u;
    for (uint32_t b = 0u; b < nb; ++b) {
        if (e.lane == 0u) blk_inc_begin(e, nb, b) = at;
        for (uint32_t base = 0u; base < tile.nheads; base += 32u) {
            const uint32_t h = base + e.lane;
            bool hit = false;
            if (h < tile.nheads) { const uint32_t o = hu(e, HF_OWNER, h); hit = (o & 0xffffu) == b || (o >> 16) == b; }
            const uint32_t m = __ballot_sync(NKB_FULL, hit);
            if (hit) inc[at + __popc(m & ((1u << e.lane) - 1u))] = h;
            at += __popc(m);
        }
    }
    if (e.lane == 0u) blk_inc_begin(e, nb, nb) = at;
    uint16_t* utab = unit_table(e, nb);
    for (uint32_t k = e.lane; k < 4u * e.vstride; k += 32u) utab[k] = (uint16_t)kNoUnitHead;
    __syncwarp();
    for (uint32_t h = e.lane; h < tile.nheads; h += 32u) {
        const uint32_t jo = hu(e, HF_JOFF, h), o = hu(e, HF_OWNER, h), fl = hu(e, HF_FLAGS, h);
        if (!(jo & kUnitRow) || ((o & 0xffffu) != e.t->B && (o >> 16) != e.t->B)) continue;
        const uint32_t slot = (fl & kHeadDrive) ? 3u : (fl & kHeadFriction) ? 2u : hf(e, HF_UNITV, h) < 0.f ? 1u : 0u;
        utab[slot * e.vstride + (jo & 0xffffu)] = (uint16_t)h;
    }
    __syncwarp();
    if (!color) return;
    uint32_t colours = 0u;       // 1 + the largest colour in use
#pragma unroll 1
    for (uint32_t b = 0u; b < nb; ++b) {
        if (blk_dim(e, b) == 0u) { if (e.lane == 0u) blk_color(e, nb, b) = 0xffffffffu; continue; }
        uint32_t taken = 0u;
        const uint32_t ib = blk_inc_begin(e, nb, b), ie = blk_inc_begin(e, nb, b + 1u);
        for (uint32_t k = ib + e.lane; k < ie; k += 32u) {
            const uint32_t o = hu(e, HF_OWNER, inc[k]);
            const uint32_t first = o & 0xffffu, second = o >> 16;
            const uint32_t other = first == b ? second : first;
            if (other < b && blk_dim(e, other) != 0u) taken |= 1u << blk_color(e, nb, other);
        }
        taken = __reduce_or_sync(NKB_FULL, taken);
        const uint32_t c = min((uint32_t)__ffs(~taken) - 1u, 31u);
        colours = max(colours, c + 1u);
        if (e.lane == 0u) blk_color(e, nb, b) = c;
        __syncwarp();
    }
    __syncwarp();
    // descent order: colour by colour, index order inside a colour (block_descent_tile.cuh:2749-2820)
    uint32_t* order = block_order(e, nb);
    uint32_t count = 0u;
#pragma unroll 1
    for (uint32_t c = 0u; c < colours; ++c)
#pragma unroll 1
        for (uint32_t base = 0u; base < nb; base += 32u) {
            const uint32_t b = base + e.lane;
            const bool hit = b < nb && blk_color(e, nb, b) == c;
            const uint32_t m = __ballot_sync(NKB_FULL, hit);
            if (hit) order[count + __popc(m & ((1u << e.lane) - 1u))] = b;
            count += __popc(m);
        }
    if (e.lane == 0u) order[nb] = count;
    __syncwarp();
}

// residual = rhs dt - J u at the blocks' current velocities (block_descent_tile.cuh:891-930)
NKB_DEV void init_residuals(Env& e, const Tile& tile) {
    const TemplateView& t = *e.t;
    const float dt = t.cfg.dt;
    for (uint32_t h = e.lane; h < tile.nheads; h += 32u) {
        const uint32_t axes = head_axes(e, h);
        V3 res = mk3(0.f, 0.f, 0.f);
        for (uint32_t ax = 0u; ax < axes; ++ax) {
            float along = 0.f;
            for (uint32_t side = 0u; side < 2u; ++side) {
                const uint32_t b = head_owner(e, h, side);
                if (b == kNoBlock16) continue;
                along += head_row_dot(e, h, side, ax, b, block_vel(e, b, false));
            }
            setc(res, (int)ax, (ax == 0u ? hf(e, HF_RHS, h) * dt : 0.f) - along);
        }
        hst3(e, HF_RES, h, res);
    }
    __syncwarp();
}

// Leading dimension of a shared-memory matrix whose rows are read as float4 by one lane per row:
// a multiple of 4 words that is 4 mod 8, so the eight lanes of a quarter warp hit distinct bank groups.
NKB_DEV uint32_t pad_ld(uint32_t n) { const uint32_t ld = (n + 3u) & ~3u; return (ld & 7u) == 0u ? ld + 4u : ld; }

// Register copy of one head for the row evaluations.
struct HeadRegs {
    V3 dual, res, move, step;
    float rho, lower, upper, rsd, rsr, mu, nb;
    bool cone;      // three-axis contact head
};
NKB_DEV HeadRegs load_head(const Env& e, uint32_t h) {
    HeadRegs r;
    r.dual = hf3(e, HF_DUAL, h); r.res = hf3(e, HF_RES, h); r.move = hf3(e, HF_MOVE, h); r.step = hf3(e, HF_STEP, h);
    r.rho = hf(e, HF_RHO, h); r.lower = hf(e, HF_LOWER, h); r.upper = hf(e, HF_UPPER, h);
    r.rsd = hf(e, HF_RSD, h); r.rsr = hf(e, HF_RSR, h); r.mu = hf(e, HF_MU, h); r.nb = hf(e, HF_NB, h);
    r.cone = head_axes(e, h) == 3u;
    return r;
}
NKB_DEV void respond(const HeadRegs& r, V3 move, V3& f, float& cxx, float& cyy, float& czz, float& cyz) {
    const Resp rs = {r.rsd, r.rsr};
    const STerm n = scalar_impulse(r.dual.x, r.rho, r.res.x - move.x, r.lower, r.upper, rs);
    f = mk3(n.impulse, 0.f, 0.f);
    cxx = n.curvature; cyy = czz = cyz = 0.f;
    if (r.cone) cone_impulse(r.dual, r.rho, r.res.y - move.y, r.res.z - move.z, r.nb, r.mu, f.y, f.z, cyy, czz, cyz);
}

// Row steps J d of a block's incident heads (block_descent_tile.cuh:2019-2044); lane = head, d staged in shared
// memory with zeros past the block's dimension.
template <bool kArtic>
NKB_DEV void row_steps(Env& e, const Tile& tile, uint32_t b, const float* dvec) {
    const uint32_t nb = tile.nblocks, dim = kArtic ? blk_dim(e, b) : 6u;
    constexpr bool artic = kArtic;
    const uint32_t* inc = blk_inc(e, nb);
    const uint32_t ib = blk_inc_begin(e, nb, b), ie = blk_inc_begin(e, nb, b + 1u);
    const uint32_t chunks = (dim + 3u) >> 2, n4 = chunks << 2;
    const float4* d4 = reinterpret_cast<const float4*>(dvec);
#pragma unroll 1
    for (uint32_t k = ib + e.lane; k < ie; k += 32u) {
        const uint32_t h = inc[k];
        const bool cone = head_axes(e, h) == 3u;
        V3 step = mk3(0.f, 0.f, 0.f);
        const uint32_t jo = hu(e, HF_JOFF, h);
        if (artic) {
            if (jo & kUnitRow) step.x = hf(e, HF_UNITV, h) * dvec[jo & 0xffffu];
            else {
                const float4* j4 = reinterpret_cast<const float4*>(sm_jpool(e) + jo);
                float s0 = 0.f, s1 = 0.f, s2 = 0.f;
#pragma unroll 1
                for (uint32_t c = 0u; c < chunks; ++c) {
                    const float4 d = d4[c], r0 = j4[c];
                    s0 = fmaf(r0.x, d.x, s0); s0 = fmaf(r0.y, d.y, s0); s0 = fmaf(r0.z, d.z, s0); s0 = fmaf(r0.w, d.w, s0);
                    if (cone) {
                        const float4 r1 = j4[chunks + c], r2 = j4[2u * chunks + c];
                        s1 = fmaf(r1.x, d.x, s1); s1 = fmaf(r1.y, d.y, s1); s1 = fmaf(r1.z, d.z, s1); s1 = fmaf(r1.w, d.w, s1);
                        s2 = fmaf(r2.x, d.x, s2); s2 = fmaf(r2.y, d.y, s2); s2 = fmaf(r2.z, d.z, s2); s2 = fmaf(r2.w, d.w, s2);
                    }
                }
                step = mk3(s0, s1, s2);
            }
        } else if (k - ib < e.lay->rjac_heads) {
            // rigid block whose head rows were staged at the start of the descent: 3 rows of 8 floats per head
            const float4* j4 = reinterpret_cast<const float4*>(e.sm + e.lay->rjac + e.newton_shift + (k - ib) * 24u);
            const float4 d0 = d4[0], d1 = d4[1];
            const float4 a0 = j4[0], a1 = j4[1];
            step.x = a0.x * d0.x + a0.y * d0.y + a0.z * d0.z + a0.w * d0.w + a1.x * d1.x + a1.y * d1.y;
            if (cone) {
                const float4 b0 = j4[2], b1 = j4[3], c0 = j4[4], c1 = j4[5];
                step.y = b0.x * d0.x + b0.y * d0.y + b0.z * d0.z + b0.w * d0.w + b1.x * d1.x + b1.y * d1.y;
                step.z = c0.x * d0.x + c0.y * d0.y + c0.z * d0.z + c0.w * d0.w + c1.x * d1.x + c1.y * d1.y;
            }
        } else {
            const uint32_t side = head_owner(e, h, 0u) == b ? 0u : 1u;
            const uint32_t axes = cone ? 3u : 1u;
#pragma unroll 1
            for (uint32_t ax = 0u; ax < axes; ++ax) {
                float s = 0.f;
#pragma unroll 1
                for (uint32_t i = 0u; i < dim; ++i) s += head_jac(e, h, side, ax, i, b) * dvec[i];
                setc(step, (int)ax, s);
            }
        }
        hst3(e, HF_STEP, h, step);
    }
    (void)n4;
    __syncwarp();
}

// One head's share of the line derivatives at step length alpha.
NKB_DEV void line_terms(const HeadRegs& r, float alpha, CSum& rs, float& rc, float& rm) {
    const V3 trial = mk3(fmaf(alpha, r.step.x, r.move.x), fmaf(alpha, r.step.y, r.move.y), fmaf(alpha, r.step.z, r.move.z));
    V3 f; float cxx, cyy, czz, cyz;
    respond(r, trial, f, cxx, cyy, czz, cyz);
    csum_addp(rs, f.x, r.step.x); csum_addp(rs, f.y, r.step.y); csum_addp(rs, f.z, r.step.z);
    rm += fabsf(f.x * r.step.x) + fabsf(f.y * r.step.y) + fabsf(f.z * r.step.z);
    rc += cxx * r.step.x * r.step.x + cyy * r.step.y * r.step.y + czz * r.step.z * r.step.z + 2.0f * cyz * r.step.y * r.step.z;
}

// Exact line search on the block's one-dimensional model (block_descent_tile.cuh:2048-2125): the first
// evaluation (alpha = 0) gives the initial slope, the following ones bracket and polish the root.  With at most
// 32 incident heads each lane keeps its head in registers for the whole search.
NKB_DEV float search_line(Env& e, const Tile& tile, uint32_t b, float islope, float icurv) {
    const uint32_t nb = tile.nblocks;
    const uint32_t* inc = blk_inc(e, nb);
    const uint32_t ib = blk_inc_begin(e, nb, b), ie = blk_inc_begin(e, nb, b + 1u);
    const bool single = ie - ib <= 32u, mine = ib + e.lane < ie;
    HeadRegs cached;
    if (single && mine) cached = load_head(e, inc[ib + e.lane]);
    float low = 0.0f, high = 0.0f, alpha = 0.0f, initial = 0.0f, result = 0.0f;
    bool bounded = false, have = false;
#pragma unroll 1
    for (int step = -1; step < (int)kLineSteps; ++step) {
        CSum rs = {0.f, 0.f};
        float rc = 0.f, rm = 0.f;
        if (single) { if (mine) line_terms(cached, alpha, rs, rc, rm); }
        else
#pragma unroll 1
        for (uint32_t k = ib + e.lane; k < ie; k += 32u) { const HeadRegs r = load_head(e, inc[k]); line_terms(r, alpha, rs, rc, rm); }
        CSum total = {-rs.value, -rs.error};
        if (e.lane == 0u) { csum_addp(total, alpha, icurv); csum_add(total, islope); }
        const float slope = warp_csum_total(total);
        const float curvature = icurv + warp_sum(rc);
        const float magnitude = fabsf(islope) + alpha * icurv + warp_sum(rm);
        if (step < 0) {
            initial = slope;
            if (!(initial < 0.0f)) { have = true; result = 0.0f; break; }
            alpha = 1.0f;
            continue;
        }
        if (!isfinite(slope) || !isfinite(curvature)) { high = alpha; bounded = true; alpha = 0.5f * (low + high); continue; }
        if (fabsf(slope) <= fmaxf(kLineTol * -initial, kRoundings * FLT_EPSILON * magnitude)) { have = true; result = alpha; break; }
        if (slope < 0.0f) low = alpha; else { high = alpha; bounded = true; }
        if (bounded && high - low <= FLT_EPSILON * high) break;
        float next = alpha - __fdividef(slope, curvature);
        if (!(next > low && (!bounded || next < high))) next = bounded ? 0.5f * (low + high) : 2.0f * alpha;
        alpha = next;
    }
    return have ? result : low;
}

NKB_DEV void apply_moves(Env& e, const Tile& tile, uint32_t b, float alpha) {
    const uint32_t nb = tile.nblocks;
    const uint32_t* inc = blk_inc(e, nb);
    const uint32_t ib = blk_inc_begin(e, nb, b), ie = blk_inc_begin(e, nb, b + 1u);
#pragma unroll 1
    for (uint32_t k = ib + e.lane; k < ie; k += 32u) {
        const uint32_t h = inc[k];
        const V3 step = hf3(e, HF_STEP, h), move = hf3(e, HF_MOVE, h);
        hst3(e, HF_MOVE, h, mk3(fmaf(alpha, step.x, move.x), fmaf(alpha, step.y, move.y), fmaf(alpha, step.z, move.z)));
    }
    __syncwarp();
}

// Newton steps with exact line search on one block.  A lane owns coordinates lane + 32 r (r < NR) and the same rows of
// the Newton matrix, which lives in the env's shared-memory slice in float4-readable rows; lane k also owns the k-th
// incident head in the row evaluations and publishes its response through the head's shared-memory fields.
// kRigid = false compiles the descent for worlds without free bodies: the articulation is the only block and the
// rigid-block code (dense 6 x 6 mass, staged 3 x 8 Jacobian rows) drops out.
// kDim = 0: the articulation's block, dimension read at run time.  kDim = 6: a free rigid body; the loops over its
// coordinates have constant bounds and unroll.  Each instance carries only its own kind's code.
template <int NR, bool kRigid, int kDim>
NKB_DEV void descend_block(Env& e, Tile& tile, uint32_t b, bool position) {
    const uint32_t l = e.lane, nb = tile.nblocks, dim = kDim != 0 ? (uint32_t)kDim : blk_dim(e, b);
    constexpr bool artic = kDim == 0;
    const uint32_t* inc = blk_inc(e, nb);
    const uint32_t ib = blk_inc_begin(e, nb, b), ie = blk_inc_begin(e, nb, b + 1u);
    // A block without a push-out row keeps its zero position correction: its descent would minimise u^T M u from u = 0.
    // (In the velocity phase an unconstrained block still has to reach its free velocity.)
    if (position && ib == ie) return;
    const uint32_t chunks = (dim + 3u) >> 2, ldh = pad_ld(dim);
    float* velocity = block_vel(e, b, position);
    float* dvec = sm_vec(e, kVecD);
    float* hi_v = sm_vec(e, kVecS0);
    float* lo_v = sm_vec(e, kVecS1);
    float* u_v = sm_vec(e, kVecS2);
    float* H = e.sm + e.lay->chol + e.newton_shift;
    float* m6 = e.sm + e.lay->bm6 + e.newton_shift;      // 6 x 12 dense mass of a rigid block, then 3 x 8 Jacobian rows of one head
    float* jscr = m6 + 72u;
    // rigid block: dense mass, and the Jacobian rows of its incident heads staged once for the whole descent
    // (3 rows of 8 floats per head, as many heads as the staging area holds)
    if (!artic) {
        if (l < 6u) {
            const float* bm = sm_bmass(e, b);
            float* row = m6 + l * 12u;
#pragma unroll
            for (uint32_t k = 0u; k < 8u; ++k) row[k] = 0.f;
            if (l < 3u) row[l] = bm[0];
            else {
                const uint32_t a = l - 3u;
                row[3u] = a == 0u ? bm[1] : a == 1u ? bm[4] : bm[5];
                row[4u] = a == 0u ? bm[4] : a == 1u ? bm[2] : bm[6];
                row[5u] = a == 0u ? bm[5] : a == 1u ? bm[6] : bm[3];
            }
        }
        if (l < 24u) jscr[l] = 0.f;
        // lane = incident head: its three rows [direction, arm x direction, 0, 0], signed by the side it sits on
        const uint32_t staged_count = min(ie - ib, e.lay->rjac_heads);      // at most 32: one pass
        if (l < staged_count) {
            const uint32_t h = inc[ib + l];
            const float sgn = head_owner(e, h, 0u) == b ? 1.f : -1.f;
            const uint32_t as = head_axes(e, h);
            const V3 arm = hf3(e, sgn > 0.f ? HF_RA : HF_RB, h);
            float4* out = reinterpret_cast<float4*>(e.sm + e.lay->rjac + e.newton_shift + l * 24u);
#pragma unroll
            for (uint32_t ax = 0u; ax < 3u; ++ax) {
                float4 lo4 = make_float4(0.f, 0.f, 0.f, 0.f), hi4 = lo4;
                if (ax < as) {
                    const V3 dir = hf3(e, ax == 0u ? HF_N : ax == 1u ? HF_T1 : HF_T2, h);
                    const V3 ang = cross(arm, dir);
                    lo4 = make_float4(sgn * dir.x, sgn * dir.y, sgn * dir.z, sgn * ang.x);
                    hi4 = make_float4(sgn * ang.y, sgn * ang.z, 0.f, 0.f);
                }
                out[2u * ax] = lo4; out[2u * ax + 1u] = hi4;
            }
        }
    }
    bool coord[NR];
    float* Hr[NR];
    const float* Mr[NR];                // this lane's rows of the block mass, zero past the block's dimension
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const uint32_t c = l + 32u * r;
        coord[r] = c < dim;
        Hr[r] = H + (coord[r] ? c : 0u) * ldh;
        Mr[r] = artic ? sm_mass(e) + (coord[r] ? c : 0u) * e.lay->ld : m6 + (coord[r] ? c : 0u) * 12u;
    }
    bool coupled = false;
    for (uint32_t k = ib + l; k < ie; k += 32u) {
        const uint32_t h = inc[k];
        const uint32_t o = hu(e, HF_OWNER, h);
        coupled |= (o & 0xffffu) != kNoBlock16 && (o >> 16) != kNoBlock16;
        hf(e, HF_NB, h) = hf(e, HF_DUAL, h);
        hst3(e, HF_MOVE, h, mk3(0.f, 0.f, 0.f));
    }
    coupled = __any_sync(NKB_FULL, coupled);
    __syncwarp();
    float start[NR], fr[NR], u[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        start[r] = coord[r] ? velocity[l + 32u * r] : 0.f;
        fr[r] = (coord[r] && !position) ? block_free(e, b)[l + 32u * r] : 0.f;
        u[r] = start[r];
    }
    bool failure = false;
    float primal = FLT_MAX;
    tick(e, 15);
    // step -1 (first velocity sweep only) is the line search toward the free velocity; steps >= 0 are Newton steps
#pragma unroll 1
    for (int step = (tile.iteration == 0u && !position) ? -1 : 0; step < (int)kNewtonSteps; ++step) {
        float d[NR], force[NR], inertia[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) { d[r] = 0.f; force[r] = 0.f; inertia[r] = 0.f; }
        if (step < 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r) d[r] = coord[r] ? fr[r] - u[r] : 0.f;
        } else {
            // ---- lane = head: responses at the current moves, published to shared memory ----
            uint32_t dense_any = 0u;
#pragma unroll 1
            for (uint32_t k = ib + l; k < ie; k += 32u) {
                const uint32_t h = inc[k];
                const HeadRegs hr = load_head(e, h);
                V3 f; float cxx, cyy, czz, cyz;
                respond(hr, hr.move, f, cxx, cyy, czz, cyz);
                const V3 noise = mk3(fabsf(f.x) + cxx * (fabsf(hr.res.x) + fabsf(hr.move.x)), fabsf(f.y) + cyy * (fabsf(hr.res.y) + fabsf(hr.move.y)),
                                     fabsf(f.z) + czz * (fabsf(hr.res.z) + fabsf(hr.move.z)));
                hst3(e, HF_F, h, f); hst3(e, HF_NZ, h, noise);
                hf(e, HF_C, h) = cxx; hf(e, HF_C + 1u, h) = cyy; hf(e, HF_C + 2u, h) = czz; hf(e, HF_C + 3u, h) = cyz;
                const bool contributes = f.x != 0.f || f.y != 0.f || f.z != 0.f || cxx != 0.f || cyy != 0.f || czz != 0.f || cyz != 0.f ||
                                         noise.x != 0.f || noise.y != 0.f || noise.z != 0.f;
                const bool unit = artic && (hu(e, HF_JOFF, h) & kUnitRow) != 0u;
                dense_any |= (contributes && !unit) ? 1u : 0u;
            }
            // ---- lane = coordinate: inertial part of H (rows of this lane) and g ----
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const float diff = u[r] - fr[r];
                const float part = diff - u[r];
                const float diff_err = (u[r] - (diff - part)) + (-fr[r] - part);
                hi_v[l + 32u * r] = diff; lo_v[l + 32u * r] = diff_err; u_v[l + 32u * r] = u[r];
            }
            __syncwarp();
            CSum inertial[NR], g[NR];
            float scale[NR], diag[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                inertial[r].value = 0.f; inertial[r].error = 0.f;
                scale[r] = 0.f; diag[r] = 0.f;
                if (coord[r]) {
                    const float4* Mr4 = reinterpret_cast<const float4*>(Mr[r]);
                    float4* Hr4 = reinterpret_cast<float4*>(Hr[r]);
#pragma unroll (kDim != 0 ? 8 : 1)
                    for (uint32_t c = 0u; c < chunks; ++c) {
                        const float4 m = Mr4[c], hi = reinterpret_cast<const float4*>(hi_v)[c], lo = reinterpret_cast<const float4*>(lo_v)[c];
                        Hr4[c] = m;
                        csum_addp(inertial[r], m.x, hi.x); inertial[r].error = fmaf(m.x, lo.x, inertial[r].error);
                        csum_addp(inertial[r], m.y, hi.y); inertial[r].error = fmaf(m.y, lo.y, inertial[r].error);
                        csum_addp(inertial[r], m.z, hi.z); inertial[r].error = fmaf(m.z, lo.z, inertial[r].error);
                        csum_addp(inertial[r], m.w, hi.w); inertial[r].error = fmaf(m.w, lo.w, inertial[r].error);
                        scale[r] += fabsf(m.x) * fabsf(hi.x) + fabsf(m.y) * fabsf(hi.y) + fabsf(m.z) * fabsf(hi.z) + fabsf(m.w) * fabsf(hi.w);
                    }
                }
                g[r].value = -inertial[r].value; g[r].error = -inertial[r].error;
            }
            tick(e, 16);
            // rows on a single coordinate only touch that coordinate (block_descent_tile.cuh:1555-1568)
            if (artic) {
                const uint16_t* utab = unit_table(e, nb);
                const uint32_t vs = e.vstride;
#pragma unroll
                for (int r = 0; r < NR; ++r) {
#pragma unroll 1
                    for (uint32_t slot = 0u; slot < 4u; ++slot) {
                        const uint32_t h = utab[slot * vs + l + 32u * r];
                        if (h == kNoUnitHead) continue;
                        const float v = hf(e, HF_UNITV, h);
                        diag[r] += v * hf(e, HF_C, h) * v;
                        csum_addp(g[r], v, hf(e, HF_F, h));
                        scale[r] += fabsf(v) * hf(e, HF_NZ, h);
                    }
                }
            }
            // dense rows: H += J^T C J, g += J^T f, one head at a time with its values broadcast from shared memory
            if (__any_sync(NKB_FULL, dense_any != 0u)) {
#pragma unroll 1
                for (uint32_t k = ib; k < ie; ++k) {
                    const uint32_t hs = inc[k];
                    const uint32_t jo = hu(e, HF_JOFF, hs);
                    if (artic && (jo & kUnitRow)) continue;
                    const V3 f = hf3(e, HF_F, hs), nz = hf3(e, HF_NZ, hs);
                    const float c0 = hf(e, HF_C, hs), c1 = hf(e, HF_C + 1u, hs), c2 = hf(e, HF_C + 2u, hs), c12 = hf(e, HF_C + 3u, hs);
                    if (!(f.x != 0.f || f.y != 0.f || f.z != 0.f || c0 != 0.f || c1 != 0.f || c2 != 0.f || c12 != 0.f || nz.x != 0.f || nz.y != 0.f || nz.z != 0.f)) continue;
                    const float* jr; uint32_t js;
                    if (artic) { jr = sm_jpool(e) + jo; js = chunks << 2; }
                    else if (k - ib < e.lay->rjac_heads) { jr = e.sm + e.lay->rjac + e.newton_shift + (k - ib) * 24u; js = 8u; }
                    else {
                        const uint32_t ss = head_owner(e, hs, 0u) == b ? 0u : 1u, as = head_axes(e, hs);
                        __syncwarp();
                        if (l < 6u) for (uint32_t ax = 0u; ax < 3u; ++ax) jscr[ax * 8u + l] = ax < as ? head_jac(e, hs, ss, ax, l, b) : 0.f;
                        __syncwarp();
                        jr = jscr; js = 8u;
                    }
                    const float4* r0 = reinterpret_cast<const float4*>(jr);
                    const float4* r1 = reinterpret_cast<const float4*>(jr + js);
                    const float4* r2 = reinterpret_cast<const float4*>(jr + 2u * js);
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        const uint32_t c = l + 32u * r;
                        const float j0 = coord[r] ? jr[c] : 0.f, j1 = coord[r] ? jr[js + c] : 0.f, j2 = coord[r] ? jr[2u * js + c] : 0.f;
                        csum_addp(g[r], j0, f.x); csum_addp(g[r], j1, f.y); csum_addp(g[r], j2, f.z);
                        scale[r] += fabsf(j0) * nz.x + fabsf(j1) * nz.y + fabsf(j2) * nz.z;
                        const float a0 = j0 * c0, a1 = j1 * c1 + j2 * c12, a2 = j2 * c2 + j1 * c12;
                        if (coord[r]) {
                            float4* Hr4 = reinterpret_cast<float4*>(Hr[r]);
#pragma unroll (kDim != 0 ? 8 : 1)
                            for (uint32_t cc = 0u; cc < chunks; ++cc) {
                                float4 h4 = Hr4[cc];
                                const float4 x = r0[cc], y = r1[cc], z = r2[cc];
                                h4.x += a0 * x.x + a1 * y.x + a2 * z.x;
                                h4.y += a0 * x.y + a1 * y.y + a2 * z.y;
                                h4.z += a0 * x.z + a1 * y.z + a2 * z.z;
                                h4.w += a0 * x.w + a1 * y.w + a2 * z.w;
                                Hr4[cc] = h4;
                            }
                        }
                    }
                }
            }
            tick(e, 17);
            bool finite = true, small = true;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                if (coord[r]) {
                    float4* Hr4 = reinterpret_cast<float4*>(Hr[r]);
                    Hr[r][l + 32u * r] += diag[r];
#pragma unroll (kDim != 0 ? 8 : 1)
                    for (uint32_t c = 0u; c < chunks; ++c) {
                        const float4 v = Hr4[c], uu = reinterpret_cast<const float4*>(u_v)[c];
                        finite &= isfinite(v.x) && isfinite(v.y) && isfinite(v.z) && isfinite(v.w);
                        scale[r] += fabsf(v.x) * fabsf(uu.x) + fabsf(v.y) * fabsf(uu.y) + fabsf(v.z) * fabsf(uu.z) + fabsf(v.w) * fabsf(uu.w);
                    }
                    force[r] = g[r].value + g[r].error; inertia[r] = inertial[r].value + inertial[r].error;
                }
                finite &= isfinite(force[r]);
                small &= !coord[r] || fabsf(force[r]) <= kRoundings * FLT_EPSILON * scale[r];
            }
            if (!__all_sync(NKB_FULL, finite)) { failure = true; break; }
            bool converged = __all_sync(NKB_FULL, small);
            if (converged && tile.tol > 0.f) {
                solve_block_mass<NR>(e, b, force, d);
                bool still = true;
#pragma unroll
                for (int r = 0; r < NR; ++r) still &= !coord[r] || fabsf(d[r]) < tile.tol;
                converged = __all_sync(NKB_FULL, still);
            }
            if (converged) { primal = 0.f; break; }
            tick(e, 18);
            // ---- Cholesky, rows of L over the rows of H (block_descent_tile.cuh:1623-1641) ----
            bool valid = true;
            float inverse[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) inverse[r] = 0.f;
            __syncwarp();
#pragma unroll (kDim != 0 ? 8 : 1)
            for (uint32_t k = 0u; k < dim; ++k) {
                float value[NR];
                const float4* Hk4 = reinterpret_cast<const float4*>(H + k * ldh);
                const uint32_t full = k >> 2, rem = k & 3u;
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    value[r] = 0.f;
                    if (coord[r] && l + 32u * r >= k) {
                        const float4* Hr4 = reinterpret_cast<const float4*>(Hr[r]);
                        float s0 = 0.f, s1 = 0.f;
#pragma unroll (kDim != 0 ? 8 : 1)
                        for (uint32_t c = 0u; c < full; ++c) {
                            const float4 a = Hr4[c], bb = Hk4[c];
                            s0 = fmaf(a.x, bb.x, s0); s1 = fmaf(a.y, bb.y, s1); s0 = fmaf(a.z, bb.z, s0); s1 = fmaf(a.w, bb.w, s1);
                        }
                        const float4 a = Hr4[full], bb = Hk4[full];
                        if (rem > 0u) s0 = fmaf(a.x, bb.x, s0);
                        if (rem > 1u) s1 = fmaf(a.y, bb.y, s1);
                        if (rem > 2u) s0 = fmaf(a.z, bb.z, s0);
                        value[r] = Hr[r][k] - (s0 + s1);
                    }
                }
                const float pivot = coord_bcast<NR>(value, k);
                valid &= pivot > 0.f && pivot <= FLT_MAX;
                const float sc = rsqrtf(valid ? pivot : 1.0f), root = pivot * sc;
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const uint32_t c = l + 32u * r;
                    if (coord[r] && c >= k) Hr[r][k] = c == k ? root : value[r] * sc;
                    inverse[r] = c == k ? sc : inverse[r];
                }
                __syncwarp();
            }
            if (!valid) { failure = true; break; }
            tick(e, 19);
            // ---- d = H^-1 g ----
            float rr[NR], scaled[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) rr[r] = force[r];
#pragma unroll (kDim != 0 ? 8 : 1)
            for (uint32_t j = 0u; j < dim; ++j) {
#pragma unroll
                for (int r = 0; r < NR; ++r) scaled[r] = rr[r] * inverse[r];
                const float y = coord_bcast<NR>(scaled, j);
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const uint32_t c = l + 32u * r;
                    rr[r] = c == j ? y : ((coord[r] && c > j) ? fmaf(-Hr[r][j], y, rr[r]) : rr[r]);
                }
            }
#pragma unroll (kDim != 0 ? 8 : 1)
            for (uint32_t jj = dim; jj > 0u; --jj) {
                const uint32_t j = jj - 1u;
#pragma unroll
                for (int r = 0; r < NR; ++r) scaled[r] = rr[r] * inverse[r];
                const float x = coord_bcast<NR>(scaled, j);
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const uint32_t c = l + 32u * r;
                    rr[r] = c == j ? x : (c < j ? fmaf(-H[j * ldh + c], x, rr[r]) : rr[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < NR; ++r) d[r] = coord[r] ? rr[r] : 0.f;
        }
        // ---- curvature and slopes along d ----
        __syncwarp();
#pragma unroll
        for (int r = 0; r < NR; ++r) dvec[l + 32u * r] = d[r];
        __syncwarp();
        CSum dec = {0.f, 0.f}, slo = {0.f, 0.f}, cur = {0.f, 0.f};
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            float ms = 0.f;
            if (coord[r]) {
                const float4* Mr4 = reinterpret_cast<const float4*>(Mr[r]);
#pragma unroll (kDim != 0 ? 8 : 1)
                for (uint32_t c = 0u; c < chunks; ++c) {
                    const float4 m = Mr4[c], dd = reinterpret_cast<const float4*>(dvec)[c];
                    ms = fmaf(m.x, dd.x, ms); ms = fmaf(m.y, dd.y, ms); ms = fmaf(m.z, dd.z, ms); ms = fmaf(m.w, dd.w, ms);
                }
                csum_addp(dec, force[r], d[r]); csum_addp(slo, inertia[r], d[r]); csum_addp(cur, d[r], ms);
            }
        }
        const float icurv = warp_csum_total(cur);
        float islope;
        if (step < 0) {
            if (!(icurv > 0.f && isfinite(icurv))) continue;
            islope = -icurv;
        } else {
            const float total_dec = warp_csum_total(dec);
            islope = warp_csum_total(slo);
            if (!isfinite(total_dec) || !isfinite(islope) || !isfinite(icurv)) { failure = true; break; }
            if (!(total_dec > 0.f)) break;
        }
        tick(e, 20);
        row_steps<artic>(e, tile, b, dvec);
        tick(e, 21);
        const float alpha = search_line(e, tile, b, islope, icurv);
        tick(e, 22);
        tick_count(e, 23);
        if (step < 0) {
            if (alpha > 0.f) {
#pragma unroll
                for (int r = 0; r < NR; ++r) u[r] = fmaf(alpha, d[r], u[r]);
                apply_moves(e, tile, b, alpha);
            }
            continue;
        }
        float after[NR];
        bool fin_l = true, rounded_l = true;
        float step_l = 0.f;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            after[r] = fmaf(alpha, d[r], u[r]);
            fin_l &= !coord[r] || isfinite(after[r]);
            rounded_l &= !coord[r] || after[r] == u[r];
            step_l = fmaxf(step_l, coord[r] ? fabsf(alpha * d[r]) : 0.f);
        }
        const bool fin = __all_sync(NKB_FULL, fin_l);
        const bool rounded = __all_sync(NKB_FULL, rounded_l);
        if (!fin) { failure = true; break; }
        primal = warp_max(rounded ? 0.f : step_l);
        if (!(alpha > 0.f)) break;
#pragma unroll
        for (int r = 0; r < NR; ++r) u[r] = after[r];
        apply_moves(e, tile, b, alpha);
        if (rounded) break;
    }
    for (uint32_t k = ib + l; k < ie; k += 32u) {
        const uint32_t h = inc[k];
        const V3 res = hf3(e, HF_RES, h), move = hf3(e, HF_MOVE, h);
        hst3(e, HF_RES, h, mk3(__fsub_rn(res.x, move.x), __fsub_rn(res.y, move.y), __fsub_rn(res.z, move.z)));
    }
    if (failure) e.status |= kStatusSolverFailure;
    float moved = failure ? FLT_MAX : 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) if (coord[r]) moved = fmaxf(moved, residual_abs(u[r] - start[r]));
    moved = warp_max(moved);
    tile.momentum = fmaxf(tile.momentum, moved);
    if (failure) primal = FLT_MAX;
    tile.residual = fmaxf(tile.residual, fmaxf(primal, coupled ? moved : 0.f));
#pragma unroll
    for (int r = 0; r < NR; ++r) if (coord[r]) velocity[l + 32u * r] = u[r];
    __syncwarp();
}

// ---- team mode: several warps on one env ---------------------------------------------------------------------------------
// Blocks of one colour share no constraint row (index_blocks colours the graph whose edges are the two-sided heads), so
// their descents touch disjoint head records and disjoint body velocities and may run side by side.  The env's lead warp
// walks the descent order; for a run of rigid blocks of one colour it publishes a command in shared memory, and every
// warp of the team (the lead included) takes the blocks member, member + team, ... of the run, each on Newton scratch of
// its own.  A result does not depend on which warp ran a block, so team sizes give bit-identical states.
//
// The warps meet through sequence numbers in shared memory, never through a hardware barrier: the lead bumps the
// command's sequence number, a helper answers by copying it into its result record.  Every wait is bounded by a cycle
// budget; a warp whose wait runs out records kStatusTeamTimeout and carries on alone (the lead descends the remaining
// blocks itself, a helper leaves), so a team that falls apart costs a status bit, not a hung kernel.
enum : uint32_t { kTeamDescend = 0x44455343u, kTeamExit = 0x45584954u,
                  // stages whose outer loop is dealt out over the team: k_begin carries the stage's count argument
                  kTeamNarrowphase = 0x4e415252u, kTeamWarmStart = 0x5741524du, kTeamCacheOwners = 0x4f574e52u };
constexpr uint32_t kTeamCommandWords = 12u;                   // the team area: command, then 4 result words per member
constexpr long long kTeamPatience = 4000000000ll;           // cycles a warp waits for another: about two seconds
struct TeamCommand { uint32_t seq, op, k_begin, k_end, position, iteration, nblocks, nheads; float tol; uint32_t dead, pad0, pad1; };
static_assert(sizeof(TeamCommand) == 4u * kTeamCommandWords, "the command occupies the first words of the team area");

NKB_DEV TeamCommand* team_command(float* sm, const SmemLayout& lay) { return reinterpret_cast<TeamCommand*>(sm + lay.team_area); }
// result record of a member: momentum, residual, status, sequence number of the last command it finished
NKB_DEV float* team_result(float* sm, const SmemLayout& lay, uint32_t member) { return sm + lay.team_area + kTeamCommandWords + 4u * member; }
NKB_DEV uint32_t team_peek(const uint32_t* word) { return *reinterpret_cast<const volatile uint32_t*>(word); }
NKB_DEV void team_poke(uint32_t* word, uint32_t value) { *reinterpret_cast<volatile uint32_t*>(word) = value; }

// Lead warp, before any helper looks: sequence numbers start at zero (called by every team's lead ahead of a block-wide
// barrier at kernel start).
NKB_DEV void team_open(float* sm, const SmemLayout& lay, uint32_t lane) {
    TeamCommand* cmd = team_command(sm, lay);
    if (lane == 0u) { cmd->seq = 0u; cmd->op = 0u; cmd->dead = 0u; }
    if (lane < lay.team) reinterpret_cast<uint32_t*>(team_result(sm, lay, lane))[3] = 0u;
}

// Lead warp: publishes a command; returns its sequence number.
NKB_DEV uint32_t team_post(float* sm, const SmemLayout& lay, uint32_t lane, uint32_t op, uint32_t k_begin, uint32_t k_end, bool position, const Tile& tile) {
    TeamCommand* cmd = team_command(sm, lay);
    __syncwarp();
    const uint32_t seq = cmd->seq + 1u;
    __syncwarp();
    if (lane == 0u) {
        cmd->op = op; cmd->k_begin = k_begin; cmd->k_end = k_end; cmd->position = position ? 1u : 0u;
        cmd->iteration = tile.iteration; cmd->nblocks = tile.nblocks; cmd->nheads = tile.nheads; cmd->tol = tile.tol;
        __threadfence_block();
        team_poke(&cmd->seq, seq);
    }
    __syncwarp();
    return seq;
}

// Lead warp: waits until every helper has answered command `seq`; false when the budget ran out.
NKB_DEV bool team_collect(float* sm, const SmemLayout& lay, uint32_t lane, uint32_t seq) {
    // every lane polls the same word, so the warp never splits over a wait
    bool answered = true;
    const long long begin = clock64();
    for (uint32_t m = 1u; m < lay.team && answered; ++m) {
        const uint32_t* done = reinterpret_cast<const uint32_t*>(team_result(sm, lay, m)) + 3;
        while (team_peek(done) != seq) {
            if (clock64() - begin > kTeamPatience) { answered = false; break; }
            __nanosleep(40);
        }
    }
    answered = __all_sync(NKB_FULL, answered);
    __threadfence_block();
    return answered;
}

// An env record for a warp that works on an env's shared-memory slice without owning its articulation lanes (a team's
// helper): pointers and lane only, no link or coordinate state.
NKB_DEV Env bare_env(float* sm, const SmemLayout* lay, const TemplateView* t, const StateView* s, uint32_t env, uint32_t lane, uint32_t vstride) {
    Env e;
    e.t = t; e.s = s; e.lay = lay; e.sm = sm; e.env = env; e.lane = lane;
    e.parent = kNoLink; e.jtype = kFixed; e.depth = 0xffffu; e.link_dof = 0u;
    e.q = e.qd = e.qdd = e.tau = 0.f;
    e.axis = mk3(0.f, 0.f, 0.f);
    e.drive_command = e.drive_dissipation = e.drive_lower = e.drive_upper = 0.f;
    e.dof_link[0] = e.dof_link[1] = 0u; e.dof_comp[0] = e.dof_comp[1] = kNoLink; e.vel0[0] = e.vel0[1] = 0.f;
    e.status = 0u; e.vstride = vstride; e.newton_shift = 0u; e.vec_shift = 0u;
#ifdef NKB_STAGE_TAPS
    e.cyc = nullptr; e.t0 = 0;
#endif
    return e;
}

// What a warp needs to descend rigid blocks, passed by value so that the function below can stay out of line without
// forcing the caller's env record into local memory.
struct RigidRun {
    float* sm;
    const SmemLayout* lay;
    const TemplateView* t;
    uint32_t lane, vstride, newton_shift, vec_shift;
    uint32_t nheads, nblocks, iteration;
    float tol;
};
struct RigidResult { float momentum, residual; uint32_t status; };

// Descends the rigid blocks order[k_begin + first], order[k_begin + first + stride], ... < k_end of one colour.
// Inlined at both call sites (the lead's and the helpers'): out of line, the layout offsets would be read through a
// pointer instead of the kernel's constant bank, which measured 30 % slower on a 48-box pile.
#ifndef NKB_RIGID_RUN_QUALIFIER
#define NKB_RIGID_RUN_QUALIFIER __forceinline__
#endif
template <bool kRigid>
__device__ NKB_RIGID_RUN_QUALIFIER RigidResult descend_rigid_run(RigidRun run, uint32_t k_begin, uint32_t k_end, uint32_t first, uint32_t stride, bool position) {
    Env e = bare_env(run.sm, run.lay, run.t, nullptr, 0u, run.lane, run.vstride);
    e.newton_shift = run.newton_shift; e.vec_shift = run.vec_shift;
    Tile tile;
    tile.nheads = run.nheads; tile.nblocks = run.nblocks; tile.iteration = run.iteration;
    tile.momentum = 0.f; tile.residual = 0.f; tile.tol = run.tol;
    const uint32_t* order = block_order(e, run.nblocks);
#pragma unroll 1
    for (uint32_t k = k_begin + first; k < k_end; k += stride) descend_block<1, kRigid, 6>(e, tile, order[k], position);
    RigidResult out;
    out.momentum = tile.momentum; out.residual = tile.residual; out.status = e.status;
    return out;
}

// Lead warp: releases the helpers for good (they need not answer).
NKB_DEV void team_dismiss(float* sm, const SmemLayout& lay, uint32_t lane) {
    if (lay.team <= 1u) return;
    Tile none;
    none.nheads = 0u; none.nblocks = 0u; none.iteration = 0u; none.momentum = 0.f; none.residual = 0.f; none.tol = 0.f;
    team_post(sm, lay, lane, kTeamExit, 0u, 0u, false, none);
}

// Lead warp: deals a stage's outer loop out over the team.  `work(first, stride)` is the loop body's range form; the lead
// runs its own share between publishing the command and collecting the answers.  Alone (no team, or a team that fell
// apart) the lead runs the whole range.  Returns the helpers' status bits.
template <typename Work>
NKB_DEV void team_fork(Env& e, uint32_t op, uint32_t count, Work&& work) {
    const uint32_t team = e.lay->team;
    if (team <= 1u || team_command(e.sm, *e.lay)->dead != 0u) { work(0u, 1u); return; }
    Tile none;
    none.nheads = 0u; none.nblocks = 0u; none.iteration = 0u; none.momentum = 0.f; none.residual = 0.f; none.tol = 0.f;
    const uint32_t seq = team_post(e.sm, *e.lay, e.lane, op, count, 0u, false, none);
    work(0u, team);
    if (team_collect(e.sm, *e.lay, e.lane, seq)) {
        for (uint32_t m = 1u; m < team; ++m) e.status |= reinterpret_cast<const uint32_t*>(team_result(e.sm, *e.lay, m))[2];
    } else {
        // a helper did not answer: flag the env, stop using the team, and do the whole range here (the stages dealt out
        // this way write each item from its inputs alone, so items done twice come out the same)
        e.status |= kStatusTeamTimeout;
        if (e.lane == 0u) team_command(e.sm, *e.lay)->dead = 1u;
        __syncwarp();
        work(0u, 1u);
    }
}

// Blocks descend colour by colour, blocks of one colour in index order (block_descent_tile.cuh:2749-2820).
template <int NR, bool kRigid>
NKB_DEV void descend_blocks(Env& e, Tile& tile, bool position) {
    const uint32_t nb = tile.nblocks;
    const uint32_t* order = block_order(e, nb);
    const uint32_t count = order[nb];
    if constexpr (!kRigid) {
#pragma unroll 1
        for (uint32_t k = 0u; k < count; ++k) descend_block<NR, false, 0>(e, tile, e.t->B, position);
    } else {
        const uint32_t team = e.lay->team;
        RigidRun run;
        run.sm = e.sm; run.lay = e.lay; run.t = e.t; run.lane = e.lane; run.vstride = e.vstride; run.newton_shift = 0u; run.vec_shift = 0u;
        run.nheads = tile.nheads; run.nblocks = nb; run.iteration = tile.iteration; run.tol = tile.tol;
#pragma unroll 1
        for (uint32_t k = 0u; k < count;) {
            const uint32_t b = order[k];
            if (b == e.t->B) { descend_block<NR, kRigid, 0>(e, tile, b, position); ++k; continue; }
            // the run of rigid blocks that share b's colour (a rigid block's 6 coordinates: one per lane)
            const uint32_t colour = blk_color(e, nb, b);
            uint32_t k_end = k + 1u;
            while (k_end < count && order[k_end] != e.t->B && blk_color(e, nb, order[k_end]) == colour) ++k_end;
            // colour 31 is the overflow colour (index_blocks hands it to every block past the 31st colour): not a set of
            // independent blocks, so it stays with the lead
            const bool shared_out = team > 1u && k_end - k > 1u && colour < 31u && team_command(e.sm, *e.lay)->dead == 0u;
            const uint32_t stride = shared_out ? team : 1u;
            uint32_t seq = 0u;
            if (shared_out) {
                seq = team_post(e.sm, *e.lay, e.lane, kTeamDescend, k, k_end, position, tile);
#ifdef NKB_STAGE_TAPS
                if (e.cyc != nullptr && e.lane == 0u) e.cyc[31] += 1u;
#endif
            }
            RigidResult mine = {0.f, 0.f, 0u};
            bool collected = true;
            uint32_t share = 0u;
            // one pass takes the lead's share (all of the run when it is not shared out); further passes only run after a
            // helper failed to answer, and take the helpers' shares
#pragma unroll 1
            do {
                const RigidResult part = descend_rigid_run<kRigid>(run, k, k_end, share, stride, position);
                mine.momentum = fmaxf(mine.momentum, part.momentum); mine.residual = fmaxf(mine.residual, part.residual);
                mine.status |= part.status;
                if (shared_out && share == 0u) {
                    collected = team_collect(e.sm, *e.lay, e.lane, seq);
                    if (collected) {
                        for (uint32_t m = 1u; m < team; ++m) {
                            const float* r = team_result(e.sm, *e.lay, m);
                            mine.momentum = fmaxf(mine.momentum, r[0]); mine.residual = fmaxf(mine.residual, r[1]);
                            mine.status |= reinterpret_cast<const uint32_t*>(r)[2];
                        }
                    } else {
                        // a helper did not answer: flag the env, stop using the team, descend the helpers' shares here
                        mine.status |= kStatusTeamTimeout;
                        if (e.lane == 0u) team_command(e.sm, *e.lay)->dead = 1u;
                        __syncwarp();
                    }
                }
                ++share;
            } while (shared_out && !collected && share < team);
            tile.momentum = fmaxf(tile.momentum, mine.momentum);
            tile.residual = fmaxf(tile.residual, mine.residual);
            e.status |= mine.status;
            k = k_end;
        }
    }
}

struct DualMomentum { float t, beta; };

// Dual update over every head (block_descent_tile.cuh:2493-2595); returns the residual classes.
NKB_DEV void update_duals(Env& e, const Tile& tile, DualMomentum* mom, bool velocity, bool commit, float out[3]) {
    float cn = 0.f, ct = 0.f, cj = 0.f;
    double restart = 0.0;
    for (uint32_t h = e.lane; h < tile.nheads; h += 32u) {
        const uint32_t fl = hu(e, HF_FLAGS, h);
        const bool contact = (fl & (kHeadContact | kHeadScalar)) == kHeadContact;
        const V3 tdual = commit ? hf3(e, HF_DUAL, h) : hf3(e, HF_BASE, h);
        const V3 res = hf3(e, HF_RES, h);
        const float rho = hf(e, HF_RHO, h), lower = hf(e, HF_LOWER, h), upper = hf(e, HF_UPPER, h), mu = hf(e, HF_MU, h);
        const Resp rs = {hf(e, HF_RSD, h), hf(e, HF_RSR, h)};
        const float normal = scalar_impulse(tdual.x, rho, res.x, lower, upper, rs).impulse;
        Relax rx;
        rx.step = hf3(e, HF_RXS, h); rx.weight = hf(e, HF_RXW, h); rx.point = hf3(e, HF_RXP, h);
        if (!commit) { rx.step = mk3(0.f, 0.f, 0.f); rx.weight = 0.f; rx.point = rx.step; }
        V3 dual;
        if (!contact) dual = mk3(normal, 0.f, 0.f);
        else {
            float iy, iz, c1, c2, c3;
            cone_impulse(tdual, rho, res.y, res.z, normal, mu, iy, iz, c1, c2, c3);
            dual = relax_contact_impulse_fast(tdual, mk3(normal, iy, iz), rx);
        }
        float sn, st;
        multiplier_steps_iso(tdual, dual, rs.residual_scale, rs.dual_scale, rho, contact ? mu : 0.f, sn, st);
        if (!commit && rs.residual_scale > 0.f) sn = __fdividef(fabsf(dual.x - tdual.x), rs.residual_scale);
        const V3 physical = commit ? dual : tdual;
        if (!contact) {
            const bool normal_row = (fl & kHeadContactNormal) != 0u;
            const float rate = -res.x;
            const float violation = physical.x > 0.f ? fabsf(rate) : fmaxf(-rate, 0.f);
            const float r = normal_row ? fmaxf(sn, violation) : sn;
            if (normal_row) cn = fmaxf(cn, residual_abs(r)); else cj = fmaxf(cj, residual_abs(r));
        } else {
            if (commit) { hst3(e, HF_RXS, h, rx.step); hf(e, HF_RXW, h) = rx.weight; hst3(e, HF_RXP, h, rx.point); }
            const V3 v = mk3(-res.x, -res.y, -res.z);
            cn = fmaxf(cn, residual_abs(physical.x > 0.f ? fabsf(v.x) : fmaxf(-v.x, 0.f)));
            ct = fmaxf(ct, residual_abs(fmaxf(st, fmaxf(along_axis(physical.y, v.y), along_axis(physical.z, v.z)))));
        }
        if (!commit) continue;
        if (velocity) hst3(e, HF_LAM, h, dual);
        const bool extrapolate = contact || rs.dual_scale != 0.f;
        const V3 base = hf3(e, HF_BASE, h);
        if (extrapolate) restart += momentum_restart_iso(tdual, dual, base, rs.residual_scale, rho, contact && mu > 0.f);
        if (mom != nullptr) hst3(e, HF_MOVE, h, base);
        hst3(e, HF_DUAL, h, dual);
        hst3(e, HF_BASE, h, dual);
    }
    __syncwarp();
    out[0] = warp_max(cn); out[1] = warp_max(ct); out[2] = warp_max(cj);
    if (mom != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) restart += __shfl_xor_sync(NKB_FULL, restart, o);
        if (restart > 0.0) mom->t = 1.0f;
        const float tn = 0.5f * (1.0f + sqrtf(fmaf(4.0f * mom->t, mom->t, 1.0f)));
        mom->beta = (mom->t - 1.0f) / tn;
        mom->t = tn;
        for (uint32_t h = e.lane; h < tile.nheads; h += 32u) {
            const bool contact = head_axes(e, h) == 3u;
            const bool extrapolate = contact || hf(e, HF_RSD, h) != 0.f;
            const float mu = hf(e, HF_MU, h);
            hst3(e, HF_DUAL, h, extrapolate_dual_iso(hf3(e, HF_MOVE, h), hf3(e, HF_BASE, h), extrapolate ? mom->beta : 0.f,
                                                     hf(e, HF_LOWER, h), hf(e, HF_UPPER, h), contact, mu));
        }
        __syncwarp();
    }
}

// Momentum balance of every moving block against the physical multipliers (block_descent_tile.cuh:2379-2489).
template <int NR, bool kRigid>
NKB_DEV void measure_primals(Env& e, Tile& tile, bool reconstruct) {
    const uint32_t nb = tile.nblocks, l = e.lane;
    const uint32_t* inc = blk_inc(e, nb);
    const uint32_t* order = block_order(e, nb);
    const uint32_t count = order[nb];
#pragma unroll 1
    for (uint32_t turn = 0u; turn < count; ++turn) {
        const uint32_t b = kRigid ? order[turn] : e.t->B;
        const uint32_t dim = blk_dim(e, b);
        const bool artic = !kRigid || b == e.t->B;
        float* vel = block_vel(e, b, false);
        const float* fr = block_free(e, b);
        const uint32_t ib = blk_inc_begin(e, nb, b), ie = blk_inc_begin(e, nb, b + 1u);
        double balance[NR];
        bool coord[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) { balance[r] = 0.0; coord[r] = l + 32u * r < dim; }
        if (artic) {
            const uint32_t n4 = (dim + 3u) & ~3u;
            const uint16_t* utab = unit_table(e, nb);
            const uint32_t vs = e.vstride;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const uint32_t c = l + 32u * r;
                if (!coord[r]) continue;
                const float* Mr = sm_mass(e) + c * e.lay->ld;
#pragma unroll 1
                for (uint32_t j = 0u; j < dim; ++j) balance[r] -= (double)Mr[j] * ((double)vel[j] - fr[j]);
#pragma unroll 1
                for (uint32_t slot = 0u; slot < 4u; ++slot) {
                    const uint32_t h = utab[slot * vs + c];
                    if (h != kNoUnitHead) balance[r] += (double)hf(e, HF_UNITV, h) * hf(e, HF_LAM, h);
                }
            }
#pragma unroll 1
            for (uint32_t k = ib; k < ie; ++k) {
                const uint32_t h = inc[k];
                const uint32_t jo = hu(e, HF_JOFF, h);
                if (jo & kUnitRow) continue;
                const V3 lam = hf3(e, HF_LAM, h);
                const float* jr = sm_jpool(e) + jo;
                const bool cone = head_axes(e, h) == 3u;
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const uint32_t c = l + 32u * r;
                    if (!coord[r]) continue;
                    balance[r] += (double)jr[c] * lam.x;
                    if (cone) balance[r] += (double)jr[n4 + c] * lam.y + (double)jr[2u * n4 + c] * lam.z;
                }
            }
        } else {
            if (coord[0]) for (uint32_t j = 0u; j < dim; ++j) balance[0] -= (double)block_mass(e, b, l, j) * ((double)vel[j] - fr[j]);
#pragma unroll 1
            for (uint32_t k = ib; k < ie; ++k) {
                const uint32_t h = inc[k];
                const uint32_t side = head_owner(e, h, 0u) == b ? 0u : 1u, axes = head_axes(e, h);
                const V3 lam = hf3(e, HF_LAM, h);
                for (uint32_t ax = 0u; ax < axes; ++ax) {
                    const float imp = comp(lam, (int)ax);
                    if (imp == 0.f) continue;
                    if (coord[0]) balance[0] += (double)head_jac(e, h, side, ax, l, b) * imp;
                }
            }
        }
        float force[NR], dir[NR];
        bool ok = true;
#pragma unroll
        for (int r = 0; r < NR; ++r) { force[r] = coord[r] ? (float)balance[r] : 0.f; dir[r] = 0.f; ok &= !coord[r] || fabs(balance[r]) <= FLT_MAX; }
        const bool finite = __all_sync(NKB_FULL, ok);
        float residual = FLT_MAX;
        if (finite) {
            solve_block_mass<NR>(e, b, force, dir);
            float worst = 0.f;
#pragma unroll
            for (int r = 0; r < NR; ++r) if (coord[r]) worst = fmaxf(worst, isfinite(dir[r]) ? fabsf(dir[r]) : FLT_MAX);
            residual = warp_max(worst);
        }
        tile.residual = fmaxf(tile.residual, residual);
        if (reconstruct && finite) {
#pragma unroll
            for (int r = 0; r < NR; ++r) if (coord[r]) vel[l + 32u * r] += dir[r];
            tile.momentum = fmaxf(tile.momentum, residual);
            __syncwarp();
        }
    }
}

// The whole constraint solve of one env.  On entry the heads are built, the articulation's post-dynamics
// velocity is in (e.qd, sm_vel(root)) and free-body velocities are in sm_bvel.
template <int NR, bool kRigid>
NKB_DEV void stage_solve(Env& e, uint32_t nheads) {
    const TemplateView& t = *e.t;
    const uint32_t l = e.lane, B = t.B, n = t.ndof;
    Tile tile;
    tile.nheads = nheads; tile.nblocks = B + (n != 0u ? 1u : 0u); tile.iteration = 0u;
    tile.momentum = tile.residual = 0.f; tile.tol = t.cfg.velocity_tolerance;
    // rigid blocks: free velocity, mass, carried constraint velocity (block_descent_rigid.cuh:4-48)
    for (uint32_t b = l; b < B; b += 32u) {
        float* bv = sm_bvel(e, b);
        float* bf = sm_bfree(e, b);
        const float im = __ldg(t.inv_mass + b);
        uint32_t dim = 0u;
        if (im > 0.f && __ldg(t.body_to_link + b) == kNoLink) {
            const float* w = sm_bwinv(e, b);
            const double xx = w[0], yy = w[1], zz = w[2], xy = w[3], xz = w[4], yz = w[5];
            const double cxx = yy * zz - yz * yz, cyy = xx * zz - xz * xz, czz = xx * yy - xy * xy;
            const double cxy = xz * yz - xy * zz, cxz = xy * yz - xz * yy, cyz = xy * xz - xx * yz;
            const double det = xx * cxx + xy * cxy + xz * cxz;
            if (det > 0.0) {
                const double inv = 1.0 / det;
                float* bm = sm_bmass(e, b);
                bm[0] = (float)(1.0 / (double)im);
                bm[1] = (float)(cxx * inv); bm[2] = (float)(cyy * inv); bm[3] = (float)(czz * inv);
                bm[4] = (float)(cxy * inv); bm[5] = (float)(cxz * inv); bm[6] = (float)(cyz * inv);
                dim = 6u;
            } else e.status |= kStatusSolverFailure;
        }
        blk_dim(e, b) = dim;
        const float* carry = e.s->carry_rigid + ((size_t)e.env * B + b) * 6u;
#pragma unroll
        for (int k = 0; k < 6; ++k) {
            bf[k] = bv[k];
            const float c = dim != 0u ? carry[k] : 0.f;
            bv[k] = bf[k] + (isfinite(c) ? c : 0.f);
        }
        float* ps = sm_bpseudo(e, b);
#pragma unroll
        for (int k = 0; k < 6; ++k) ps[k] = 0.f;
    }
    if (n != 0u && l == 0u) blk_dim(e, B) = n;
    // articulation coordinates: free = post-dynamics velocity
    {
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint32_t at = l + 32u * r;
            const float qd_of_link = __shfl_sync(NKB_FULL, e.qd, e.dof_link[r]);
            if (at < n) {
                const float value = e.dof_comp[r] == kNoLink ? qd_of_link : sm_vel(e, e.dof_link[r])[e.dof_comp[r]];
                const float c = e.s->carry_artic[(size_t)e.env * n + at];
                sm_vec(e, kVecFree)[at] = value;
                sm_vec(e, kVecU)[at] = value + (isfinite(c) ? c : 0.f);
                sm_vec(e, kVecPseudo)[at] = 0.f;
            } else { sm_vec(e, kVecFree)[at] = 0.f; sm_vec(e, kVecU)[at] = 0.f; sm_vec(e, kVecPseudo)[at] = 0.f; }   // float4 readers see zeros past n
        }
    }
    __syncwarp();
    init_heads<NR>(e, tile);
    tick(e, 8);
    float rows[3] = {0.f, 0.f, 0.f};
    float cls[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t sweeps = 0u, positions = 0u, pushes = 0u;
    DualMomentum mom = {1.0f, 0.0f};
    const uint32_t iterations = t.cfg.vel_iters;
    // One loop drives the velocity sweeps, the hand-over and the split-impulse position sweeps so that each of
    // the large pieces (block indexing, block descent, dual update, momentum balance) is instantiated once.
    enum { kPhaseVelocity, kPhaseHandOver, kPhasePosition, kPhaseDone };
    int phase = kPhaseVelocity;
    bool reindex = true;
    while (phase != kPhaseDone) {
        if (reindex) {
            index_blocks(e, tile, phase == kPhaseVelocity);
            reindex = false;
            if (phase == kPhaseVelocity) { init_residuals(e, tile); tick(e, 9); if (iterations == 0u) phase = kPhaseHandOver; }
        }
        if (phase == kPhaseHandOver) {
            if (l < 4u) e.s->solver_residual[(size_t)e.env * 4u + l] = cls[l];
            if (l == 0u) e.s->solver_sweeps[e.env] = sweeps;
            // velocities back to the links, carried velocities to global memory
            if (n != 0u) {
                const float* U = sm_vec(e, kVecU);
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const uint32_t at = l + 32u * r;
                    if (at < n) {
                        e.s->carry_artic[(size_t)e.env * n + at] = U[at] - sm_vec(e, kVecFree)[at];
                        if (e.dof_comp[r] != kNoLink) sm_vel(e, e.dof_link[r])[e.dof_comp[r]] = U[at];
                    }
                }
                if (l < t.L && joint_dofs(e.jtype) == 1u) e.qd = U[e.link_dof];
            }
            for (uint32_t b = l; b < B; b += 32u) {
                float* carry = e.s->carry_rigid + ((size_t)e.env * B + b) * 6u;
                const float* bv = sm_bvel(e, b);
                const float* bf = sm_bfree(e, b);
#pragma unroll
                for (int k = 0; k < 6; ++k) carry[k] = blk_dim(e, b) != 0u ? bv[k] - bf[k] : 0.f;
            }
            __syncwarp();
            phase = kPhaseDone;
            // split-impulse position pass: every head becomes a scalar push-out row (ops/block_descent.cu:1734-1753)
            if (t.cfg.pos_iters != 0u && nheads != 0u) {
                bool push = false, coupled = false;
                for (uint32_t h = l; h < nheads; h += 32u) {
                    const uint32_t fl = hu(e, HF_FLAGS, h);
                    const bool spec = (fl & kHeadSpeculative) != 0u;
                    const float slop = spec ? 0.f : t.cfg.pos_slop;
                    const float pen_row = hf(e, HF_PEN, h);
                    const bool active = (fl & kHeadVelocityOnly) == 0u && (spec || pen_row > slop || hf(e, HF_DUAL, h) != 0.f);
                    float bias = 0.f, rounding = 0.f;
                    if (active) {
                        const float penetration = fmaxf(pen_row - slop, 0.f);
                        if (spec) {
                            const float cd = sm_cdepth(e)[hu(e, HF_REF, h) & 0xffffu];
                            const double depth = (double)cd - slop, reserve = (double)pen_row - cd;
                            const double correction = t.cfg.pos_beta * fmax(depth, 0.0) + reserve;
                            const double target = fmin(depth, 0.0) + correction;
                            double velocity = 0.0;
                            for (uint32_t side = 0u; side < 2u; ++side) {
                                const uint32_t b = head_owner(e, h, side);
                                if (b == kNoBlock16) continue;
                                velocity += (double)head_row_dot(e, h, side, 0u, b, block_vel(e, b, false));
                            }
                            const double limit = fmin(correction / t.cfg.dt, (double)t.cfg.baumgarte_max_velocity);
                            bias = (float)fmin(target / t.cfg.dt - velocity, limit);
                            rounding = (float)(target > 0.0 ? 0.0 : fmax(reserve, 0.0) / t.cfg.dt);
                        } else {
                            bias = fminf(t.cfg.pos_beta * penetration / t.cfg.dt, t.cfg.baumgarte_max_velocity);
                        }
                    } else hu(e, HF_OWNER, h) = kNoBlock16 | (kNoBlock16 << 16);
                    const uint32_t o = hu(e, HF_OWNER, h);
                    coupled |= (o & 0xffffu) != kNoBlock16 && (o >> 16) != kNoBlock16;
                    hu(e, HF_FLAGS, h) = fl | kHeadScalar;
                    hf(e, HF_LOWER, h) = 0.f; hf(e, HF_UPPER, h) = FLT_MAX;
                    const Resp rs = scalar_response(hf(e, HF_RHO, h), 0.f);
                    hf(e, HF_RSD, h) = rs.dual_scale; hf(e, HF_RSR, h) = rs.residual_scale;
                    hst3(e, HF_RES, h, mk3(bias, 0.f, 0.f));
                    hst3(e, HF_DUAL, h, mk3(0.f, 0.f, 0.f));
                    push |= bias > rounding;
                }
                push = __any_sync(NKB_FULL, push); coupled = __any_sync(NKB_FULL, coupled);
                __syncwarp();
                if (push) { phase = kPhasePosition; reindex = true; positions = coupled ? t.cfg.pos_iters : 1u; pushes = 0u; }
            }
            continue;
        }
        if (phase == kPhaseVelocity) { tile.iteration = sweeps++; tile.momentum = 0.f; tile.residual = 0.f; }
        else tile.iteration = sweeps + pushes;
        descend_blocks<NR, kRigid>(e, tile, phase == kPhasePosition);
        if (phase == kPhasePosition) {
            if (++pushes >= positions) { phase = kPhaseDone; continue; }
        } else tick(e, 10);
        update_duals(e, tile, phase == kPhaseVelocity ? &mom : nullptr, phase == kPhaseVelocity, true, rows);
        if (phase == kPhasePosition) continue;
        tick(e, 24);
        // momentum balance: plain measure, reconstruction when only the primal lags, re-measure after it
        for (int stage = 0; stage < 3; ++stage) {
            const float worst_row = fmaxf(fmaxf(rows[0], rows[1]), rows[2]);
            bool run = true;
            if (stage == 0) run = sweeps == iterations || fmaxf(worst_row, tile.residual) < tile.tol;
            else if (stage == 1) run = worst_row < tile.tol && tile.residual >= tile.tol && tile.residual < FLT_MAX;
            if (stage == 1 && !run) break;
            if (run) { measure_primals<NR, kRigid>(e, tile, stage == 1); tick(e, 25); tick_count(e, 27); }
            if (stage == 1) {
                if (!(tile.residual < FLT_MAX)) break;
                init_residuals(e, tile);
                update_duals(e, tile, nullptr, true, false, rows);
                tile.residual = 0.f;
                tick(e, 26);
            }
        }
        cls[0] = rows[0]; cls[1] = rows[1]; cls[2] = rows[2]; cls[3] = tile.residual;
        const float largest = fmaxf(fmaxf(rows[0], rows[1]), fmaxf(rows[2], tile.residual));
        tick(e, 11);
        if (sweeps >= iterations || largest < tile.tol || largest == FLT_MAX) phase = kPhaseHandOver;
    }
    tick(e, 14);
    if (e.s->dbg_qdot_pseudo != nullptr) for (uint32_t at = l; at < n; at += 32u) e.s->dbg_qdot_pseudo[(size_t)e.env * n + at] = sm_vec(e, kVecPseudo)[at];
}

}  // namespace nkb
