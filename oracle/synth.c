/*
 * CPU twin of the library's synthetic-input recipe — TEST INFRASTRUCTURE.
 *
 * Generates, on the host cores, the same R-MAT CSR and the same feature table
 * the GPU generators (aethergraph_b200/csrc/synth.cu) produce for a given seed,
 * so the CPU baseline can run without a GPU and both sides can be checked
 * against each other.  The recipe (pure integer arithmetic on the SplitMix64
 * finalizer) is stated at the top of synth.cu; rows are sorted by
 * (source, destination), which makes the result independent of how the edges
 * were produced.
 */
#define _GNU_SOURCE
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define G1 0x9E3779B97F4A7C15ULL
#define G2 0xD6E8FEB86659FD93ULL

static inline uint64_t mix(uint64_t x) {
    uint64_t z = x + G1;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

static inline float unit_normal(uint64_t seed, uint64_t e) {
    const uint64_t r0 = mix(seed ^ mix(e)), r1 = mix(r0 + G1);
    uint32_t s = 0;
    for (int k = 0; k < 4; ++k) s += (uint32_t)((r0 >> (16 * k)) & 0xFFFF) + (uint32_t)((r1 >> (16 * k)) & 0xFFFF);
    return (float)((int)s - 262140) * 1.8688173e-05f;
}

typedef struct {
    uint64_t num_src, num_dst, num_edges, seed;
    uint32_t bits_src, bits_dst, a16, ab16, abc16;
} rmat_params;

static uint32_t bits_for(uint64_t n) { uint32_t b = 0; while ((1ULL << b) < n) ++b; return b; }

static inline void rmat_edge(const rmat_params *p, uint64_t i, uint32_t *s, uint32_t *d) {
    const uint64_t base = mix(p->seed ^ mix(i));
    const uint32_t levels = p->bits_src > p->bits_dst ? p->bits_src : p->bits_dst;
    for (uint32_t t = 0;; ++t) {
        const uint64_t st = mix(base + (uint64_t)t * G1);
        uint64_t src = 0, dst = 0, word = 0;
        for (uint32_t l = 0; l < levels; ++l) {
            if ((l & 3u) == 0) word = mix(st + (uint64_t)(l / 4 + 1) * G2);
            const uint32_t u = (uint32_t)(word >> (16 * (l & 3u))) & 0xFFFFu;
            const uint32_t sb = u >= p->ab16 ? 1u : 0u;
            const uint32_t db = ((u >= p->a16 && u < p->ab16) || u >= p->abc16) ? 1u : 0u;
            if (l + p->bits_src >= levels) src = (src << 1) | sb;
            if (l + p->bits_dst >= levels) dst = (dst << 1) | db;
        }
        if (src < p->num_src && dst < p->num_dst) { *s = (uint32_t)src; *d = (uint32_t)dst; return; }
        if (t == 63) { *s = (uint32_t)(src % p->num_src); *d = (uint32_t)(dst % p->num_dst); return; }
    }
}

static int cmp_u32(const void *a, const void *b) {
    const uint32_t x = *(const uint32_t *)a, y = *(const uint32_t *)b;
    return x < y ? -1 : x > y;
}

static void sort_row(uint32_t *r, uint64_t n) {
    if (n < 2) return;
    if (n <= 24) { /* insertion sort: the common case */
        for (uint64_t i = 1; i < n; ++i) {
            uint32_t v = r[i]; uint64_t j = i;
            while (j > 0 && r[j - 1] > v) { r[j] = r[j - 1]; --j; }
            r[j] = v;
        }
        return;
    }
    qsort(r, n, 4, cmp_u32);
}

/* Fills offsets (num_src + 1, caller-allocated) and dst (num_edges, caller-allocated). */
int ago_synth_rmat_csr(uint64_t num_src, uint64_t num_dst, uint64_t num_edges, float a, float b, float c,
                       uint64_t seed, int threads, uint64_t *offsets, uint32_t *dst) {
    if (!num_src || !num_dst) return -1;
    rmat_params p;
    p.num_src = num_src; p.num_dst = num_dst; p.num_edges = num_edges; p.seed = seed;
    p.bits_src = bits_for(num_src); p.bits_dst = bits_for(num_dst);
    p.a16 = (uint32_t)(a * 65536.0f);
    p.ab16 = (uint32_t)((a + b) * 65536.0f);
    p.abc16 = (uint32_t)((a + b + c) * 65536.0f);
    if (threads < 1) threads = 1;
    uint32_t *deg = (uint32_t *)calloc(num_src + 1, 4);
    if (!deg) return -2;
    /* pass 1: out-degrees */
#pragma omp parallel for num_threads(threads) schedule(static)
    for (uint64_t i = 0; i < num_edges; ++i) {
        uint32_t s, d;
        rmat_edge(&p, i, &s, &d);
        __atomic_fetch_add(&deg[s], 1u, __ATOMIC_RELAXED);
    }
    offsets[0] = 0;
    for (uint64_t v = 0; v < num_src; ++v) offsets[v + 1] = offsets[v] + deg[v];
    memset(deg, 0, (num_src + 1) * 4);
    /* pass 2: scatter (order within a row is fixed by the sort below) */
#pragma omp parallel for num_threads(threads) schedule(static)
    for (uint64_t i = 0; i < num_edges; ++i) {
        uint32_t s, d;
        rmat_edge(&p, i, &s, &d);
        const uint32_t at = __atomic_fetch_add(&deg[s], 1u, __ATOMIC_RELAXED);
        dst[offsets[s] + at] = d;
    }
    free(deg);
#pragma omp parallel for num_threads(threads) schedule(dynamic, 4096)
    for (uint64_t v = 0; v < num_src; ++v) sort_row(dst + offsets[v], offsets[v + 1] - offsets[v]);
    return 0;
}

static inline uint16_t enc_bf16(float v) {
    uint32_t bits; memcpy(&bits, &v, 4);
    return (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
}

uint16_t ago_f32_to_f16(float v);

/* Rows [row_begin, row_end) of the synthetic table, encoded as dtype (0 f32, 1 f16, 2 bf16). */
int ago_synth_features(uint64_t dim, int dtype, uint64_t seed, uint64_t row_begin, uint64_t row_end,
                       int threads, void *payload) {
    const uint64_t total = (row_end - row_begin) * dim, first = row_begin * dim;
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(static)
    for (uint64_t g = 0; g < total; ++g) {
        const float f = unit_normal(seed, first + g);
        if (dtype == 0) ((float *)payload)[g] = f;
        else if (dtype == 2) ((uint16_t *)payload)[g] = enc_bf16(f);
        else ((uint16_t *)payload)[g] = ago_f32_to_f16(f);
    }
    return 0;
}
