/*
 * CPU oracle — TEST INFRASTRUCTURE, NOT PRODUCT CODE (see oracle.h).
 * Plain C restatement of the reference's CPU minibatch path.
 */
#define _GNU_SOURCE
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ======================================================================
 * RNG
 * ==================================================================== */

/* sampler.rs:69-75 — SplitMix64 finalizer over base ^ idx * golden ratio. */
uint64_t ago_batch_seed(uint64_t base, uint64_t batch_idx) {
    uint64_t z = base ^ (batch_idx * 0x9E3779B97F4A7C15ULL);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

/* genstamp.rs:192-196 */
static inline uint64_t wy_mix(uint64_t state) {
    __uint128_t t = (__uint128_t)state * (__uint128_t)(state ^ 0xe7037ed1a0b428dbULL);
    return (uint64_t)((t >> 64) ^ t);
}

uint64_t ago_wyrand_next_u64(ago_wyrand *r) {
    r->state += 0xa0761d6478bd642fULL;
    return wy_mix(r->state);
}

/* genstamp.rs:199-201 */
uint32_t ago_wyrand_next_u32(ago_wyrand *r) {
    return (uint32_t)ago_wyrand_next_u64(r);
}

uint64_t ago_wyrand_at(uint64_t seed, uint64_t d) {
    return wy_mix(seed + (d + 1) * 0xa0761d6478bd642fULL);
}

/* philox.rs:15-40 */
void ago_philox4x32_10(uint64_t seed, uint32_t layer, uint64_t node,
                       uint32_t draw_group, uint32_t out[4]) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
    const uint32_t W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
    uint32_t c0 = (uint32_t)node, c1 = (uint32_t)(node >> 32), c2 = layer, c3 = draw_group;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    for (int round = 0; round < 10; ++round) {
        uint64_t p0 = (uint64_t)c0 * M0, p1 = (uint64_t)c2 * M1;
        uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
        uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
        uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        if (round != 9) { k0 += W0; k1 += W1; }
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* philox.rs:43-52 */
uint32_t ago_philox_u32(uint64_t seed, uint32_t layer, uint64_t node,
                        uint32_t draw_index) {
    uint32_t r[4];
    ago_philox4x32_10(seed, layer, node, draw_index >> 2, r);
    return r[draw_index & 3];
}

/* philox.rs:59-82 — Algorithm R keyed by the scan position t. */
size_t ago_reservoir_sample(const uint32_t *neighbors, size_t degree,
                            size_t fanout, uint64_t seed, uint32_t layer,
                            uint64_t node, uint32_t *out) {
    if (degree == 0 || fanout == 0) return 0;
    if (fanout >= degree) {
        memcpy(out, neighbors, degree * sizeof(uint32_t));
        return degree;
    }
    memcpy(out, neighbors, fanout * sizeof(uint32_t));
    for (size_t t = fanout; t < degree; ++t) {
        uint32_t r = ago_philox_u32(seed, layer, node, (uint32_t)t);
        size_t j = (size_t)r % (t + 1);
        if (j < fanout) out[j] = neighbors[t];
    }
    return fanout;
}

/* sampler.rs:52-55 */
double ago_neg_ln_u64(uint64_t bits) {
    double u = ((double)(bits >> 11) + 1.0) * (1.0 / 9007199254740992.0);
    return -log(u);
}

/* ======================================================================
 * Feature codecs
 * ==================================================================== */

static inline uint32_t f32_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static inline float bits_f32(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

/* store.rs:1094-1104 */
uint16_t ago_f32_to_bf16(float v) {
    uint32_t bits = f32_bits(v);
    if (v != v) return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t bias = 0x7FFFu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + bias) >> 16);
}

/* IEEE binary32 -> binary16, round to nearest even. */
uint16_t ago_f32_to_f16(float v) {
    uint32_t x = f32_bits(v);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 0xFFu) { /* inf / nan: keep nan quiet with its top payload bits */
        if (man == 0) return (uint16_t)(sign | 0x7C00u);
        return (uint16_t)(sign | 0x7C00u | 0x0200u | (man >> 13));
    }
    int32_t e = (int32_t)exp - 127 + 15;
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u); /* overflow -> inf */
    if (e <= 0) {
        /* subnormal half or zero */
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);            /* 14..24 */
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++; /* may carry into exp */
    return (uint16_t)(sign | half);
}

/* simd.rs:233-238 */
float ago_bf16_to_f32(uint16_t bits) { return bits_f32((uint32_t)bits << 16); }

/* half::f16::to_f32 (simd.rs:97-101): exact widening. */
float ago_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0x1Fu) {
        /* A NaN keeps its payload and comes out quiet: what half 2.x's software
         * path and the F16C / AVX-512 converts the reference dispatches to
         * (simd.rs:57-95) all produce. */
        if (man) return bits_f32(sign | 0x7FC00000u | (man << 13));
        return bits_f32(sign | 0x7F800000u);
    }
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* normalise the subnormal */
        int shift = 0;
        while (!(man & 0x400u)) { man <<= 1; ++shift; }
        man &= 0x3FFu;
        uint32_t e = (uint32_t)(127 - 15 - shift + 1);
        return bits_f32(sign | (e << 23) | (man << 13));
    }
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

void ago_encode_rows(const float *src, size_t count, int dtype, void *dst) {
    if (dtype == AGO_F32) { memcpy(dst, src, count * 4); return; }
    uint16_t *d = (uint16_t *)dst;
    if (dtype == AGO_F16) for (size_t i = 0; i < count; ++i) d[i] = ago_f32_to_f16(src[i]);
    else for (size_t i = 0; i < count; ++i) d[i] = ago_f32_to_bf16(src[i]);
}

void ago_decode_rows(const void *src, size_t count, int dtype, float *dst) {
    if (dtype == AGO_F32) { memcpy(dst, src, count * 4); return; }
    const uint16_t *s = (const uint16_t *)src;
    if (dtype == AGO_F16) for (size_t i = 0; i < count; ++i) dst[i] = ago_f16_to_f32(s[i]);
    else for (size_t i = 0; i < count; ++i) dst[i] = ago_bf16_to_f32(s[i]);
}

static inline size_t elem_size(int dtype) { return dtype == AGO_F32 ? 4 : 2; }

/* header.rs:110-116 */
static inline void decode_row(const uint8_t *src, float *dst, size_t dim, int dtype) {
    if (dtype == AGO_F32) { memcpy(dst, src, dim * 4); return; }
    const uint16_t *s = (const uint16_t *)src;
    if (dtype == AGO_BF16) for (size_t j = 0; j < dim; ++j) dst[j] = ago_bf16_to_f32(s[j]);
    else for (size_t j = 0; j < dim; ++j) dst[j] = ago_f16_to_f32(s[j]);
}

/* store.rs:777-838: validate every id, then decode row nodes[i] into out[i]
 * with a software prefetch a fixed byte window ahead (store.rs:320-330). */
int64_t ago_gather(const void *payload, uint64_t num_nodes, uint64_t dim,
                   int dtype, const uint32_t *ids, size_t n, float *out) {
    for (size_t i = 0; i < n; ++i)
        if ((uint64_t)ids[i] >= num_nodes) return -1 - (int64_t)i;
    const uint8_t *raw = (const uint8_t *)payload;
    size_t row_bytes = (size_t)dim * elem_size(dtype);
    size_t ahead = (8u << 10) / (row_bytes ? row_bytes : 1);
    if (ahead < 1) ahead = 1;
    if (ahead > 16) ahead = 16;
    for (size_t i = 0; i < n; ++i) {
        if (i + ahead < n) {
            const uint8_t *p = raw + (size_t)ids[i + ahead] * row_bytes;
            for (size_t o = 0; o < row_bytes; o += 64) __builtin_prefetch(p + o, 0, 0);
        }
        decode_row(raw + (size_t)ids[i] * row_bytes, out + i * dim, dim, dtype);
    }
    return 0;
}

/* ======================================================================
 * Block-scaled int8 feature codec (internal/feature_codec.rs:73-133)
 * ==================================================================== */
/* encode_rows: per 32-element block of a row, scale = max|x| / 127 (0 for an
 * all-zero block, whose codes stay 0), code = round(x / scale) clamped to
 * [-127, 127] (f32::round: half away from zero).  Returns -1 for a value that is
 * not finite (FeatureCodecError::NotFinite), -2 for dim == 0. */
int ago_encode_i8(const float *values, size_t rows, size_t dim, int8_t *codes, float *scales) {
    if (dim == 0) return -2;
    size_t per_row = (dim + 31) / 32;
    memset(codes, 0, rows * dim);
    for (size_t row = 0; row < rows; ++row) {
        const float *src = values + row * dim;
        for (size_t b = 0; b < per_row; ++b) {
            size_t lo = b * 32, hi = lo + 32 < dim ? lo + 32 : dim;
            float peak = 0.0f;
            for (size_t i = lo; i < hi; ++i) {
                if (!isfinite(src[i])) return -1;
                float a = fabsf(src[i]);
                if (a > peak) peak = a;
            }
            float scale = peak == 0.0f ? 0.0f : peak / 127.0f;
            scales[row * per_row + b] = scale;
            if (scale == 0.0f) continue;
            for (size_t i = lo; i < hi; ++i) {
                float q = roundf(src[i] / scale);
                if (q < -127.0f) q = -127.0f;
                if (q > 127.0f) q = 127.0f;
                codes[row * dim + i] = (int8_t)q;
            }
        }
    }
    return 0;
}

/* decode_into (feature_codec.rs:121-133) of the rows `ids`, in ids order:
 * out[i][e] = (float)codes[ids[i]][e] * scales[ids[i]][e / 32]. */
int64_t ago_gather_i8(const int8_t *codes, const float *scales, uint64_t num_nodes, uint64_t dim,
                      const uint32_t *ids, size_t n, float *out) {
    for (size_t i = 0; i < n; ++i)
        if ((uint64_t)ids[i] >= num_nodes) return -1 - (int64_t)i;
    size_t per_row = (dim + 31) / 32;
    for (size_t i = 0; i < n; ++i) {
        const int8_t *c = codes + (size_t)ids[i] * dim;
        const float *sc = scales + (size_t)ids[i] * per_row;
        for (size_t e = 0; e < dim; ++e) out[i * dim + e] = (float)c[e] * sc[e / 32];
    }
    return 0;
}

/* ======================================================================
 * CRC32 (IEEE 802.3, reflected, poly 0xEDB88320) — mmap.rs:642-652
 * ==================================================================== */
uint32_t ago_crc32(uint32_t crc, const void *data, size_t len) {
    static uint32_t table[256];
    static int ready = 0;
    if (!ready) {
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t c = i;
            for (int k = 0; k < 8; ++k) c = (c & 1u) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
            table[i] = c;
        }
        ready = 1;
    }
    const uint8_t *p = (const uint8_t *)data;
    crc = ~crc;
    for (size_t i = 0; i < len; ++i) crc = table[(crc ^ p[i]) & 0xFFu] ^ (crc >> 8);
    return ~crc;
}

/* ======================================================================
 * Dedup: dense generation-stamped slots or a map (genstamp.rs:33-130).
 * Both give the same answers; the map here is open addressing with a
 * touched-slot list so a pass resets in O(entries).
 * ==================================================================== */
typedef struct {
    int dense;
    /* dense */
    uint64_t *slots; uint64_t len; uint32_t generation;
    /* map */
    uint64_t *tab; uint64_t cap; uint64_t count;
    uint64_t *touched; uint64_t touched_cap;
} dedup_t;

#define MAP_EMPTY 0xFFFFFFFFFFFFFFFFULL

static void dedup_init(dedup_t *d, uint64_t num_nodes, uint64_t dense_max) {
    memset(d, 0, sizeof *d);
    if (num_nodes <= dense_max) {
        d->dense = 1;
        d->len = num_nodes;
        d->slots = (uint64_t *)calloc(num_nodes ? num_nodes : 1, 8);
    } else {
        d->cap = 1024;
        d->tab = (uint64_t *)malloc(d->cap * 8);
        memset(d->tab, 0xFF, d->cap * 8);
        d->touched_cap = 1024;
        d->touched = (uint64_t *)malloc(d->touched_cap * 8);
    }
}

static void dedup_destroy(dedup_t *d) { free(d->slots); free(d->tab); free(d->touched); }

/* genstamp.rs:55-61, 99-104 */
static void dedup_begin(dedup_t *d) {
    if (d->dense) {
        d->generation += 1;
        if (d->generation == 0) { memset(d->slots, 0, d->len * 8); d->generation = 1; }
    } else {
        for (uint64_t i = 0; i < d->count; ++i) d->tab[d->touched[i]] = MAP_EMPTY;
        d->count = 0;
    }
}

static inline uint64_t map_hash(uint32_t key, uint64_t mask) {
    return ((uint64_t)key * 0x9E3779B97F4A7C15ULL >> 20) & mask;
}

static void map_grow(dedup_t *d) {
    uint64_t ncap = d->cap * 2;
    uint64_t *nt = (uint64_t *)malloc(ncap * 8);
    memset(nt, 0xFF, ncap * 8);
    uint64_t *ntouched = (uint64_t *)malloc(ncap * 8);
    uint64_t c = 0;
    for (uint64_t i = 0; i < d->count; ++i) {
        uint64_t e = d->tab[d->touched[i]];
        uint64_t h = map_hash((uint32_t)(e >> 32), ncap - 1);
        while (nt[h] != MAP_EMPTY) h = (h + 1) & (ncap - 1);
        nt[h] = e;
        ntouched[c++] = h;
    }
    free(d->tab); free(d->touched);
    d->tab = nt; d->touched = ntouched; d->cap = ncap; d->touched_cap = ncap;
}

/* genstamp.rs:63-75, 109-120: returns the local index; *inserted says whether
 * `global` was new and got `next_local`. */
static inline uint32_t dedup_probe_or_insert(dedup_t *d, uint32_t global,
                                             uint32_t next_local, int *inserted) {
    if (d->dense) {
        uint64_t slot = d->slots[global];
        if ((uint32_t)(slot >> 32) == d->generation) { *inserted = 0; return (uint32_t)slot; }
        d->slots[global] = ((uint64_t)d->generation << 32) | next_local;
        *inserted = 1;
        return next_local;
    }
    if ((d->count + 1) * 2 > d->cap) map_grow(d);
    uint64_t mask = d->cap - 1, h = map_hash(global, mask);
    for (;;) {
        uint64_t e = d->tab[h];
        if (e == MAP_EMPTY) {
            d->tab[h] = ((uint64_t)global << 32) | next_local;
            d->touched[d->count++] = h;
            *inserted = 1;
            return next_local;
        }
        if ((uint32_t)(e >> 32) == global) { *inserted = 0; return (uint32_t)e; }
        h = (h + 1) & mask;
    }
}

/* ======================================================================
 * Growable arrays
 * ==================================================================== */
typedef struct { uint32_t *p; size_t n, cap; } vec32;
typedef struct { uint64_t *p; size_t n, cap; } vec64;

static inline void v32_push(vec32 *v, uint32_t x) {
    if (v->n == v->cap) { v->cap = v->cap ? v->cap * 2 : 1024; v->p = (uint32_t *)realloc(v->p, v->cap * 4); }
    v->p[v->n++] = x;
}
static inline void v64_push(vec64 *v, uint64_t x) {
    if (v->n == v->cap) { v->cap = v->cap ? v->cap * 2 : 1024; v->p = (uint64_t *)realloc(v->p, v->cap * 8); }
    v->p[v->n++] = x;
}
/* Hands the array to the caller and leaves a fresh one of capacity `next_cap`
 * behind (0: none) — the swap with a planned-capacity vector of
 * sampler.rs:897-924, so the next batch does not regrow from nothing. */
static uint32_t *v32_take(vec32 *v, size_t next_cap) {
    uint32_t *p = v->p ? v->p : (uint32_t *)malloc(4);
    v->p = next_cap ? (uint32_t *)malloc(next_cap * 4) : NULL;
    v->n = 0; v->cap = v->p ? next_cap : 0; return p;
}
static uint64_t *v64_take(vec64 *v, size_t next_cap) {
    uint64_t *p = v->p ? v->p : (uint64_t *)malloc(8);
    v->p = next_cap ? (uint64_t *)malloc(next_cap * 8) : NULL;
    v->n = 0; v->cap = v->p ? next_cap : 0; return p;
}
/* loader/mod.rs:27-29 */
static inline size_t planned_capacity(size_t produced, size_t floor) {
    size_t c = produced + produced / 8;
    return c > floor ? c : floor;
}

/* Floyd membership for one node's draws (sampler.rs:1342-1379).  The
 * reference uses a 256-entry stamp block for n <= 256 and a hash set above;
 * the two are the same set.  Here: the stamp block, plus a linear list for
 * larger rows (k picks, k small relative to the row). */
typedef struct {
    uint32_t stamp[256]; uint32_t generation;
    uint64_t *list; size_t n, cap;
} floyd_t;

static void floyd_begin(floyd_t *f) {
    f->generation += 1;
    if (f->generation == 0) { memset(f->stamp, 0, sizeof f->stamp); f->generation = 1; }
    f->n = 0;
}
/* returns 1 when i was not yet taken (and marks it) */
static int floyd_test_and_set(floyd_t *f, size_t row_len, uint64_t i) {
    if (row_len <= 256) {
        if (f->stamp[i] != f->generation) { f->stamp[i] = f->generation; return 1; }
        return 0;
    }
    for (size_t k = 0; k < f->n; ++k) if (f->list[k] == i) return 0;
    if (f->n == f->cap) { f->cap = f->cap ? f->cap * 2 : 64; f->list = (uint64_t *)realloc(f->list, f->cap * 8); }
    f->list[f->n++] = i;
    return 1;
}

/* ======================================================================
 * Homogeneous sampler
 * ==================================================================== */
typedef struct { double key; uint64_t idx; } wkey_t;

struct ago_sampler {
    ago_csr g;
    uint32_t *fanout; uint32_t num_hops;
    int replace, weighted, track_edge_ids;
    ago_wyrand rng;
    uint64_t draws;
    dedup_t dedup;
    vec32 nodes, edge_src, edge_dst, src_local, dst_local, seed_locals;
    vec64 edge_ids;
    vec32 fr_id, fr_local, nf_id, nf_local; /* frontiers carry (global id, local) */
    floyd_t floyd;
    wkey_t *wkeys; size_t wkeys_cap;
};

ago_sampler *ago_sampler_new(const ago_csr *g, const ago_config *cfg) {
    ago_sampler *s = (ago_sampler *)calloc(1, sizeof *s);
    s->g = *g;
    s->num_hops = cfg->num_hops;
    s->fanout = (uint32_t *)malloc(4 * (cfg->num_hops ? cfg->num_hops : 1));
    memcpy(s->fanout, cfg->fanout, 4 * cfg->num_hops);
    s->replace = cfg->replace;
    /* sampler.rs:767-771: weights are used only when configured AND present */
    s->weighted = cfg->weighted && g->weights != NULL;
    s->track_edge_ids = cfg->track_edge_ids;
    s->rng.state = cfg->seed; /* genstamp.rs:187-189 */
    uint64_t dense_max = cfg->dense_dedup_max_nodes ? cfg->dense_dedup_max_nodes : (8ULL << 20);
    dedup_init(&s->dedup, g->num_nodes, dense_max); /* sampler.rs:455-465 */
    return s;
}

void ago_sampler_free(ago_sampler *s) {
    if (!s) return;
    dedup_destroy(&s->dedup);
    free(s->fanout);
    free(s->nodes.p); free(s->edge_src.p); free(s->edge_dst.p); free(s->src_local.p);
    free(s->dst_local.p); free(s->seed_locals.p); free(s->edge_ids.p);
    free(s->fr_id.p); free(s->fr_local.p); free(s->nf_id.p); free(s->nf_local.p);
    free(s->floyd.list); free(s->wkeys);
    free(s);
}

void ago_sampler_reseed(ago_sampler *s, uint64_t seed) { s->rng.state = seed; }

/* sampler.rs:1059-1061 */
static inline uint64_t rand_below(ago_sampler *s, uint64_t n) {
    s->draws++;
    return ((uint64_t)ago_wyrand_next_u32(&s->rng) * n) >> 32;
}

/* sampler.rs:715-729 (no times) */
static inline uint32_t reg_node(ago_sampler *s, uint32_t id, int *is_new) {
    uint32_t idx = dedup_probe_or_insert(&s->dedup, id, (uint32_t)s->nodes.n, is_new);
    if (*is_new) v32_push(&s->nodes, id);
    return idx;
}

/* sampler.rs:1277-1285 + 736-745 + 1262-1270 */
static inline void emit_edge(ago_sampler *s, uint32_t src, uint32_t src_local,
                             uint32_t neighbor, uint64_t eid) {
    if ((uint64_t)neighbor >= s->g.num_nodes) return; /* corrupt destination skipped */
    int is_new;
    uint32_t dl = reg_node(s, neighbor, &is_new);
    if (is_new) { v32_push(&s->nf_id, neighbor); v32_push(&s->nf_local, dl); }
    v32_push(&s->edge_src, src);
    v32_push(&s->edge_dst, neighbor);
    v32_push(&s->src_local, src_local);
    v32_push(&s->dst_local, dl);
    if (s->track_edge_ids) v64_push(&s->edge_ids, eid);
}

static int wkey_cmp(const void *a, const void *b) {
    const wkey_t *x = (const wkey_t *)a, *y = (const wkey_t *)b;
    if (x->key < y->key) return -1;
    if (x->key > y->key) return 1;
    return x->idx < y->idx ? -1 : (x->idx > y->idx);
}

/* sampler.rs:1418-1469.  Selection follows the reference (n draws in row
 * order, key = -ln(u)/w in f64, +inf for non-finite or non-positive weight,
 * k smallest keys win).  Emission ORDER of the k winners is this oracle's own
 * (ascending key, ties by row position): the reference's comes from
 * select_nth_unstable_by and is not reproducible from its tree. */
static void sample_weighted(ago_sampler *s, uint32_t node, uint32_t node_local,
                            const uint32_t *nb, const float *w, uint64_t n,
                            uint64_t edge_offset, uint64_t k) {
    if (k == 0) return;
    if (k >= n) {
        for (uint64_t i = 0; i < n; ++i) emit_edge(s, node, node_local, nb[i], edge_offset + i);
        return;
    }
    if (s->wkeys_cap < n) { s->wkeys_cap = n * 2; s->wkeys = (wkey_t *)realloc(s->wkeys, s->wkeys_cap * sizeof(wkey_t)); }
    for (uint64_t i = 0; i < n; ++i) {
        uint64_t bits = ago_wyrand_next_u64(&s->rng);
        s->draws++;
        double wd = (double)w[i];
        double key = (isfinite(wd) && wd > 0.0) ? ago_neg_ln_u64(bits) / wd : INFINITY;
        s->wkeys[i].key = key; s->wkeys[i].idx = i;
    }
    qsort(s->wkeys, n, sizeof(wkey_t), wkey_cmp);
    for (uint64_t t = 0; t < k; ++t) {
        uint64_t idx = s->wkeys[t].idx;
        emit_edge(s, node, node_local, nb[idx], edge_offset + idx);
    }
}

/* sampler.rs:1383-1412: cumulative weights summed in f64 in row order, then k
 * draws u = next_u64 * (total / u64::MAX), each picking the first position whose
 * cumulative weight exceeds u (partition_point(c <= u), clamped to the last). */
static void sample_weighted_replace(ago_sampler *s, uint32_t node, uint32_t node_local,
                                    const uint32_t *nb, const float *w, uint64_t n,
                                    uint64_t edge_offset, uint64_t k) {
    if (n == 0) return;
    if (s->wkeys_cap < n) { s->wkeys_cap = n * 2; s->wkeys = (wkey_t *)realloc(s->wkeys, s->wkeys_cap * sizeof(wkey_t)); }
    double total = 0.0;
    for (uint64_t i = 0; i < n; ++i) { total += (double)w[i]; s->wkeys[i].key = total; }
    double scale = total / 18446744073709551615.0; /* u64::MAX as f64 */
    for (uint64_t t = 0; t < k; ++t) {
        uint64_t bits = ago_wyrand_next_u64(&s->rng);
        s->draws++;
        double u = (double)bits * scale;
        uint64_t lo = 0, hi = n; /* partition_point: first i with !(c_i <= u) */
        while (lo < hi) {
            uint64_t mid = lo + (hi - lo) / 2;
            if (s->wkeys[mid].key <= u) lo = mid + 1; else hi = mid;
        }
        uint64_t idx = lo < n - 1 ? lo : n - 1;
        emit_edge(s, node, node_local, nb[idx], edge_offset + idx);
    }
}

/* sampler.rs:1178-1235 (no hub cap: max_degree is None on this path) */
static void sample_normal(ago_sampler *s, uint32_t node, uint32_t node_local,
                          const uint32_t *nb, const float *w, uint64_t n,
                          uint64_t edge_offset, uint64_t k) {
    if (w) {
        if (s->replace) sample_weighted_replace(s, node, node_local, nb, w, n, edge_offset, k);
        else sample_weighted(s, node, node_local, nb, w, n, edge_offset, k);
        return;
    }
    if (s->replace) { /* sampler.rs:1289-1308 */
        for (uint64_t t = 0; t < k; ++t) {
            uint64_t idx = rand_below(s, n);
            emit_edge(s, node, node_local, nb[idx], edge_offset + idx);
        }
    } else if (k >= n) { /* sampler.rs:1312-1328 */
        for (uint64_t i = 0; i < n; ++i) emit_edge(s, node, node_local, nb[i], edge_offset + i);
    } else { /* sampler.rs:1332-1380 */
        floyd_begin(&s->floyd);
        for (uint64_t i = n - k; i < n; ++i) {
            uint64_t j = rand_below(s, i + 1);
            uint64_t pick;
            if (floyd_test_and_set(&s->floyd, n, j)) pick = j;
            else { floyd_test_and_set(&s->floyd, n, i); pick = i; }
            emit_edge(s, node, node_local, nb[pick], edge_offset + pick);
        }
    }
}

int64_t ago_sample(ago_sampler *s, const uint32_t *seeds, size_t n, ago_subgraph *out) {
    memset(out, 0, sizeof *out);
    /* sampler.rs:230-239 */
    for (size_t i = 0; i < n; ++i)
        if ((uint64_t)seeds[i] >= s->g.num_nodes) return -1 - (int64_t)i;

    /* sampler.rs:694-707 */
    dedup_begin(&s->dedup);
    s->nodes.n = s->edge_src.n = s->edge_dst.n = s->src_local.n = s->dst_local.n = 0;
    s->seed_locals.n = 0; s->edge_ids.n = 0;
    s->fr_id.n = s->fr_local.n = s->nf_id.n = s->nf_local.n = 0;
    uint64_t draws_before = s->draws;

    /* sampler.rs:865-872 */
    for (size_t i = 0; i < n; ++i) {
        int is_new;
        uint32_t local = reg_node(s, seeds[i], &is_new);
        v32_push(&s->seed_locals, local);
        if (is_new) { v32_push(&s->fr_id, seeds[i]); v32_push(&s->fr_local, local); }
    }

    out->num_hops = s->num_hops;
    out->num_sampled_nodes = (uint64_t *)calloc(s->num_hops + 1, 8);
    out->num_sampled_edges = (uint64_t *)calloc(s->num_hops ? s->num_hops : 1, 8);
    out->num_sampled_nodes[0] = s->nodes.n; /* sampler.rs:876-878 */

    /* sampler.rs:754-842 */
    for (uint32_t hop = 0; hop < s->num_hops; ++hop) {
        size_t edges_before = s->edge_src.n;
        uint64_t k = s->fanout[hop];
        s->nf_id.n = s->nf_local.n = 0;
        size_t flen = s->fr_id.n;
        for (size_t fi = 0; fi < flen; ++fi) {
            /* sampler.rs:786-800: the offsets pair of the vertex 4 ahead and the row
             * start of the vertex 2 ahead (FRONTIER_PREFETCH_DIST = 4, genstamp.rs:23) */
            if (fi + 4 < flen) {
                uint64_t ahead = s->fr_id.p[fi + 4];
                if (ahead < s->g.num_nodes) __builtin_prefetch(&s->g.offsets[ahead], 0, 3);
            }
            if (fi + 2 < flen) {
                uint64_t ahead = s->fr_id.p[fi + 2];
                if (ahead < s->g.num_nodes) {
                    uint64_t st = s->g.offsets[ahead];
                    if (st < s->g.num_edges) __builtin_prefetch(&s->g.edges[st], 0, 3);
                }
            }
            uint32_t node = s->fr_id.p[fi], node_local = s->fr_local.p[fi];
            /* csr.rs:318-335 */
            if ((uint64_t)node >= s->g.num_nodes) continue;
            uint64_t start = s->g.offsets[node], end = s->g.offsets[node + 1];
            if (start > end || end > s->g.num_edges) continue;
            if (start == end) continue;
            const float *w = s->weighted ? s->g.weights + start : NULL;
            sample_normal(s, node, node_local, s->g.edges + start, w, end - start, start, k);
        }
        out->num_sampled_nodes[hop + 1] = s->nf_id.n;        /* sampler.rs:827-831 */
        out->num_sampled_edges[hop] = s->edge_src.n - edges_before;
        /* sampler.rs:839: swap frontiers */
        vec32 t;
        t = s->fr_id; s->fr_id = s->nf_id; s->nf_id = t;
        t = s->fr_local; s->fr_local = s->nf_local; s->nf_local = t;
    }

    out->num_nodes = s->nodes.n; out->num_edges = s->edge_src.n; out->num_seeds = n;
    /* sampler.rs:897-924: each array is swapped for one sized from what this call
     * produced (MIN_NODE_CAPACITY 512, MIN_EDGE_CAPACITY 2048, sampler.rs:410-411) */
    const size_t ncap = planned_capacity(s->nodes.n, 512), ecap = planned_capacity(s->edge_src.n, 2048);
    out->nodes = v32_take(&s->nodes, ncap);
    out->edge_src = v32_take(&s->edge_src, ecap);
    out->edge_dst = v32_take(&s->edge_dst, ecap);
    out->src_local = v32_take(&s->src_local, ecap);
    out->dst_local = v32_take(&s->dst_local, ecap);
    out->seed_locals = v32_take(&s->seed_locals, n ? n : 1);
    if (s->track_edge_ids) out->edge_ids = v64_take(&s->edge_ids, ecap);
    out->draws = s->draws - draws_before;
    return 0;
}

void ago_subgraph_free(ago_subgraph *sg) {
    free(sg->nodes); free(sg->edge_src); free(sg->edge_dst); free(sg->edge_ids);
    free(sg->src_local); free(sg->dst_local); free(sg->seed_locals);
    free(sg->num_sampled_nodes); free(sg->num_sampled_edges);
    memset(sg, 0, sizeof *sg);
}

/* ======================================================================
 * Heterogeneous sampler
 * ==================================================================== */

/* hetero.rs:70-97: stable counting-sort transpose; rows past num_src and
 * destinations past num_dst are dropped. */
void ago_transpose(const ago_csr *csr, uint64_t num_src, uint64_t num_dst,
                   ago_in_adjacency *out) {
    uint64_t rows = csr->num_nodes < num_src ? csr->num_nodes : num_src;
    uint64_t *offsets = (uint64_t *)calloc(num_dst + 1, 8);
    for (uint64_t s = 0; s < rows; ++s) {
        uint64_t a = csr->offsets[s], b = csr->offsets[s + 1];
        if (a > b || b > csr->num_edges) continue; /* csr.rs:318-335 */
        for (uint64_t e = a; e < b; ++e) {
            uint64_t d = csr->edges[e];
            if (d < num_dst) offsets[d + 1] += 1;
        }
    }
    for (uint64_t i = 1; i <= num_dst; ++i) offsets[i] += offsets[i - 1];
    uint64_t *cursor = (uint64_t *)malloc((num_dst ? num_dst : 1) * 8);
    memcpy(cursor, offsets, num_dst * 8);
    uint32_t *sources = (uint32_t *)malloc((offsets[num_dst] ? offsets[num_dst] : 1) * 4);
    for (uint64_t s = 0; s < rows; ++s) {
        uint64_t a = csr->offsets[s], b = csr->offsets[s + 1];
        if (a > b || b > csr->num_edges) continue;
        for (uint64_t e = a; e < b; ++e) {
            uint64_t d = csr->edges[e];
            if (d < num_dst) sources[cursor[d]++] = (uint32_t)s;
        }
    }
    free(cursor);
    out->offsets = offsets; out->sources = sources; out->num_dst = num_dst;
}

void ago_in_adjacency_free(ago_in_adjacency *a) {
    free(a->offsets); free(a->sources); memset(a, 0, sizeof *a);
}

struct ago_hetero_sampler {
    uint32_t nt, et, num_hops;
    uint64_t *num_nodes;
    uint32_t *src_type, *dst_type;
    uint32_t *fanout; /* [et][hop] */
    int replace;
    ago_wyrand rng; uint64_t draws;
    ago_in_adjacency *in_adj;
    dedup_t *dedup;      /* per node type */
    vec32 *nodes;        /* per node type */
    vec32 *esrc, *edst;  /* per edge type */
    vec32 fr_type, fr_id, fr_local, nf_type, nf_id, nf_local;
    vec32 seed_indices;
    floyd_t floyd;
};

ago_hetero_sampler *ago_hetero_sampler_new(const ago_hetero_config *cfg) {
    ago_hetero_sampler *s = (ago_hetero_sampler *)calloc(1, sizeof *s);
    s->nt = cfg->num_node_types; s->et = cfg->num_edge_types; s->num_hops = cfg->num_hops;
    s->num_nodes = (uint64_t *)malloc(8 * (s->nt ? s->nt : 1));
    memcpy(s->num_nodes, cfg->num_nodes, 8 * s->nt);
    s->src_type = (uint32_t *)malloc(4 * (s->et ? s->et : 1));
    s->dst_type = (uint32_t *)malloc(4 * (s->et ? s->et : 1));
    s->fanout = (uint32_t *)malloc(4 * (size_t)(s->et ? s->et : 1) * (s->num_hops ? s->num_hops : 1));
    memcpy(s->fanout, cfg->fanout, 4 * (size_t)s->et * s->num_hops);
    s->replace = cfg->replace;
    s->rng.state = cfg->seed;
    s->in_adj = (ago_in_adjacency *)calloc(s->et ? s->et : 1, sizeof(ago_in_adjacency));
    for (uint32_t e = 0; e < s->et; ++e) {
        s->src_type[e] = cfg->relations[e].src_type;
        s->dst_type[e] = cfg->relations[e].dst_type;
        /* hetero.rs:409-423 */
        ago_transpose(&cfg->relations[e].csr, s->num_nodes[s->src_type[e]],
                      s->num_nodes[s->dst_type[e]], &s->in_adj[e]);
    }
    uint64_t dense_max = cfg->dense_dedup_max_nodes ? cfg->dense_dedup_max_nodes : (1ULL << 20);
    s->dedup = (dedup_t *)calloc(s->nt ? s->nt : 1, sizeof(dedup_t));
    for (uint32_t t = 0; t < s->nt; ++t) dedup_init(&s->dedup[t], s->num_nodes[t], dense_max);
    s->nodes = (vec32 *)calloc(s->nt ? s->nt : 1, sizeof(vec32));
    s->esrc = (vec32 *)calloc(s->et ? s->et : 1, sizeof(vec32));
    s->edst = (vec32 *)calloc(s->et ? s->et : 1, sizeof(vec32));
    return s;
}

void ago_hetero_sampler_free(ago_hetero_sampler *s) {
    if (!s) return;
    for (uint32_t e = 0; e < s->et; ++e) { ago_in_adjacency_free(&s->in_adj[e]); free(s->esrc[e].p); free(s->edst[e].p); }
    for (uint32_t t = 0; t < s->nt; ++t) { dedup_destroy(&s->dedup[t]); free(s->nodes[t].p); }
    free(s->in_adj); free(s->dedup); free(s->nodes); free(s->esrc); free(s->edst);
    free(s->num_nodes); free(s->src_type); free(s->dst_type); free(s->fanout);
    free(s->fr_type.p); free(s->fr_id.p); free(s->fr_local.p);
    free(s->nf_type.p); free(s->nf_id.p); free(s->nf_local.p);
    free(s->seed_indices.p); free(s->floyd.list);
    free(s);
}

void ago_hetero_sampler_reseed(ago_hetero_sampler *s, uint64_t seed) { s->rng.state = seed; }

const ago_in_adjacency *ago_hetero_in_adjacency(const ago_hetero_sampler *s, uint32_t edge_type) {
    return &s->in_adj[edge_type];
}

/* hetero_sampler.rs:335-342 */
static inline uint32_t h_insert_node(ago_hetero_sampler *s, uint32_t id, uint32_t type, int *is_new) {
    uint32_t idx = dedup_probe_or_insert(&s->dedup[type], id, (uint32_t)s->nodes[type].n, is_new);
    if (*is_new) v32_push(&s->nodes[type], id);
    return idx;
}

/* hetero_sampler.rs:348-355 */
static inline void h_emit(ago_hetero_sampler *s, uint32_t src_id, uint32_t src_type,
                          uint32_t dst_local, uint32_t et) {
    int is_new;
    uint32_t sl = h_insert_node(s, src_id, src_type, &is_new);
    if (is_new) { v32_push(&s->nf_type, src_type); v32_push(&s->nf_id, src_id); v32_push(&s->nf_local, sl); }
    v32_push(&s->esrc[et], sl);
    v32_push(&s->edst[et], dst_local);
}

/* hetero_sampler.rs:359-361 */
static inline uint64_t h_rand_below(ago_hetero_sampler *s, uint64_t n) {
    s->draws++;
    return ((uint64_t)ago_wyrand_next_u32(&s->rng) * n) >> 32;
}

int64_t ago_hetero_sample(ago_hetero_sampler *s, uint32_t seed_type,
                          const uint32_t *seeds, size_t n, ago_hetero_subgraph *out) {
    memset(out, 0, sizeof *out);
    for (size_t i = 0; i < n; ++i)
        if ((uint64_t)seeds[i] >= s->num_nodes[seed_type]) return -1 - (int64_t)i;

    /* hetero_sampler.rs:199-212 */
    for (uint32_t t = 0; t < s->nt; ++t) { dedup_begin(&s->dedup[t]); s->nodes[t].n = 0; }
    for (uint32_t e = 0; e < s->et; ++e) { s->esrc[e].n = 0; s->edst[e].n = 0; }
    s->fr_type.n = s->fr_id.n = s->fr_local.n = 0;
    s->seed_indices.n = 0;
    uint64_t draws_before = s->draws;

    /* hetero_sampler.rs:217-223 */
    for (size_t i = 0; i < n; ++i) {
        int is_new;
        uint32_t idx = h_insert_node(s, seeds[i], seed_type, &is_new);
        v32_push(&s->seed_indices, idx);
        if (is_new) { v32_push(&s->fr_type, seed_type); v32_push(&s->fr_id, seeds[i]); v32_push(&s->fr_local, idx); }
    }

    /* hetero_sampler.rs:228-289 */
    for (uint32_t hop = 0; hop < s->num_hops; ++hop) {
        s->nf_type.n = s->nf_id.n = s->nf_local.n = 0;
        size_t flen = s->fr_id.n;
        for (size_t fi = 0; fi < flen; ++fi) {
            uint32_t ntype = s->fr_type.p[fi], id = s->fr_id.p[fi], dst_local = s->fr_local.p[fi];
            /* incoming edge types in ascending edge-type id (hetero.rs:396-403) */
            for (uint32_t et = 0; et < s->et; ++et) {
                if (s->dst_type[et] != ntype) continue;
                uint64_t fanout = s->fanout[(size_t)et * s->num_hops + hop];
                if (fanout == 0) continue;
                const ago_in_adjacency *a = &s->in_adj[et];
                if ((uint64_t)id >= a->num_dst) continue; /* hetero.rs:99-106 */
                uint64_t start = a->offsets[id], end = a->offsets[id + 1];
                uint64_t len = end - start;
                if (len == 0) continue;
                const uint32_t *sources = a->sources + start;
                uint32_t st = s->src_type[et];
                if (s->replace) { /* hetero_sampler.rs:371-383 */
                    for (uint64_t t = 0; t < fanout; ++t)
                        h_emit(s, sources[h_rand_below(s, len)], st, dst_local, et);
                } else if (len <= fanout) { /* :364-368 */
                    for (uint64_t i = 0; i < len; ++i) h_emit(s, sources[i], st, dst_local, et);
                } else { /* :386-422 */
                    floyd_begin(&s->floyd);
                    for (uint64_t i = len - fanout; i < len; ++i) {
                        uint64_t j = h_rand_below(s, i + 1);
                        uint64_t pick;
                        if (floyd_test_and_set(&s->floyd, len, j)) pick = j;
                        else { floyd_test_and_set(&s->floyd, len, i); pick = i; }
                        h_emit(s, sources[pick], st, dst_local, et);
                    }
                }
            }
        }
        vec32 t;
        t = s->fr_type; s->fr_type = s->nf_type; s->nf_type = t;
        t = s->fr_id; s->fr_id = s->nf_id; s->nf_id = t;
        t = s->fr_local; s->fr_local = s->nf_local; s->nf_local = t;
    }

    out->num_node_types = s->nt; out->num_edge_types = s->et;
    out->nodes = (uint32_t **)calloc(s->nt ? s->nt : 1, sizeof(uint32_t *));
    out->num_nodes = (size_t *)calloc(s->nt ? s->nt : 1, sizeof(size_t));
    out->edge_src_local = (uint32_t **)calloc(s->et ? s->et : 1, sizeof(uint32_t *));
    out->edge_dst_local = (uint32_t **)calloc(s->et ? s->et : 1, sizeof(uint32_t *));
    out->num_edges = (size_t *)calloc(s->et ? s->et : 1, sizeof(size_t));
    for (uint32_t t = 0; t < s->nt; ++t) { out->num_nodes[t] = s->nodes[t].n; out->nodes[t] = v32_take(&s->nodes[t], planned_capacity(s->nodes[t].n, 0)); }
    for (uint32_t e = 0; e < s->et; ++e) {
        out->num_edges[e] = s->esrc[e].n;
        out->edge_src_local[e] = v32_take(&s->esrc[e], planned_capacity(s->esrc[e].n, 0));
        out->edge_dst_local[e] = v32_take(&s->edst[e], planned_capacity(s->edst[e].n, 0));
    }
    out->num_seeds = n;
    out->seed_indices = v32_take(&s->seed_indices, n ? n : 1);
    out->draws = s->draws - draws_before;
    return 0;
}

void ago_hetero_subgraph_free(ago_hetero_subgraph *sg) {
    for (uint32_t t = 0; t < sg->num_node_types; ++t) free(sg->nodes[t]);
    for (uint32_t e = 0; e < sg->num_edge_types; ++e) { free(sg->edge_src_local[e]); free(sg->edge_dst_local[e]); }
    free(sg->nodes); free(sg->num_nodes); free(sg->edge_src_local); free(sg->edge_dst_local);
    free(sg->num_edges); free(sg->seed_indices);
    memset(sg, 0, sizeof *sg);
}

/* ======================================================================
 * Timed CPU baseline
 * ==================================================================== */
static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

int ago_bench_run(const ago_csr *g, const ago_config *cfg,
                  const void *payload, uint64_t dim, int dtype,
                  const uint32_t *seeds, size_t batch_size, size_t num_batches,
                  uint64_t first_position, int threads, ago_bench_result *res) {
    memset(res, 0, sizeof *res);
    if (threads < 1) threads = 1;
#ifndef _OPENMP
    threads = 1;
#endif
    ago_sampler **samplers = (ago_sampler **)calloc((size_t)threads, sizeof(ago_sampler *));
    float **bufs = (float **)calloc((size_t)threads, sizeof(float *));
    size_t *buf_rows = (size_t *)calloc((size_t)threads, sizeof(size_t));
    for (int t = 0; t < threads; ++t) samplers[t] = ago_sampler_new(g, cfg);

    uint64_t edges = 0, nodes = 0, checksum = 0;
    int failed = 0;
    double t0 = now_s();
#ifdef _OPENMP
#pragma omp parallel for num_threads(threads) schedule(dynamic, 1) reduction(+ : edges, nodes) reduction(^ : checksum) reduction(| : failed)
#endif
    for (size_t b = 0; b < num_batches; ++b) {
        int tid = 0;
#ifdef _OPENMP
        tid = omp_get_thread_num();
#endif
        ago_sampler *s = samplers[tid];
        ago_sampler_reseed(s, ago_batch_seed(cfg->seed, first_position + b));
        ago_subgraph sg;
        if (ago_sample(s, seeds + b * batch_size, batch_size, &sg) != 0) { failed |= 1; continue; }
        edges += sg.num_edges; nodes += sg.num_nodes;
        uint64_t c = sg.num_edges * 0x9E3779B97F4A7C15ULL + sg.num_nodes;
        if (sg.num_edges) c ^= (uint64_t)sg.edge_dst[sg.num_edges - 1] << 17 ^ sg.dst_local[sg.num_edges - 1];
        if (payload) {
            if (buf_rows[tid] < sg.num_nodes) {
                free(bufs[tid]);
                buf_rows[tid] = sg.num_nodes + sg.num_nodes / 8;
                bufs[tid] = (float *)malloc(buf_rows[tid] * dim * 4);
            }
            if (ago_gather(payload, g->num_nodes, dim, dtype, sg.nodes, sg.num_nodes, bufs[tid]) != 0) failed |= 1;
            else if (sg.num_nodes) {
                uint32_t bits; memcpy(&bits, &bufs[tid][(sg.num_nodes - 1) * dim], 4);
                c ^= (uint64_t)bits << 7;
            }
        }
        checksum ^= c * (b + 1);
        ago_subgraph_free(&sg);
    }
    double t1 = now_s();
    for (int t = 0; t < threads; ++t) { ago_sampler_free(samplers[t]); free(bufs[t]); }
    free(samplers); free(bufs); free(buf_rows);
    res->batches = num_batches; res->edges = edges; res->nodes = nodes;
    res->seconds = t1 - t0; res->threads = threads; res->checksum = checksum;
    return failed ? -1 : 0;
}
