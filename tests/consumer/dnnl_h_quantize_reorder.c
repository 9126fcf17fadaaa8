/* A plain C program written against the reference library's C header (dnnl.h), linked against
 * libonednn_b200.so: quantise a 64 x 256 f32 tensor to s8 with one scale per row through
 * dnnl_reorder with a scales attribute, data moved with dnnl_memory_map_data.
 * Prints "OK <impl>" and exits 0, or a message and a non-zero code.
 * TEST INFRASTRUCTURE: built by oracle/build_ref.py where the reference headers are present. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "oneapi/dnnl/dnnl.h"

#define CK(x) \
    do { \
        dnnl_status_t s_ = (x); \
        if (s_ != dnnl_success) { \
            printf("%s failed with status %d\n", #x, (int)s_); \
            return 1; \
        } \
    } while (0)

int main(void) {
    enum { R = 64, C = 256 };
    static float src[R * C], scale[R];
    static int8_t got[R * C];
    unsigned seed = 12345u;
    for (int i = 0; i < R * C; ++i) {
        seed = seed * 1664525u + 1013904223u;
        src[i] = ((float)(seed >> 8) / 8388608.f - 1.f) * (1.f + (float)(i / C) * 0.1f);
    }
    for (int r = 0; r < R; ++r) {
        float amax = 0.f;
        for (int c = 0; c < C; ++c) amax = fmaxf(amax, fabsf(src[r * C + c]));
        scale[r] = amax / 127.f;
    }

    dnnl_engine_t eng;
    dnnl_stream_t strm;
    CK(dnnl_engine_create(&eng, dnnl_gpu, 0));
    CK(dnnl_stream_create(&strm, eng, dnnl_stream_default_flags));
    const dnnl_dims_t dims = {R, C}, sdims = {R};
    dnnl_memory_desc_t src_md, dst_md, sc_md;
    CK(dnnl_memory_desc_create_with_tag(&src_md, 2, dims, dnnl_f32, dnnl_ab));
    CK(dnnl_memory_desc_create_with_tag(&dst_md, 2, dims, dnnl_s8, dnnl_ab));
    CK(dnnl_memory_desc_create_with_tag(&sc_md, 1, sdims, dnnl_f32, dnnl_a));
    dnnl_primitive_attr_t attr;
    CK(dnnl_primitive_attr_create(&attr));
    CK(dnnl_primitive_attr_set_scales_mask(attr, DNNL_ARG_DST, 1 << 0));
    dnnl_primitive_desc_t pd;
    CK(dnnl_reorder_primitive_desc_create(&pd, src_md, eng, dst_md, eng, attr));
    const char *impl = NULL;
    CK(dnnl_primitive_desc_query(pd, dnnl_query_impl_info_str, 0, &impl));
    dnnl_primitive_t prim;
    CK(dnnl_primitive_create(&prim, pd));

    dnnl_memory_t src_m, dst_m, sc_m;
    CK(dnnl_memory_create(&src_m, src_md, eng, DNNL_MEMORY_ALLOCATE));
    CK(dnnl_memory_create(&dst_m, dst_md, eng, DNNL_MEMORY_ALLOCATE));
    CK(dnnl_memory_create(&sc_m, sc_md, eng, DNNL_MEMORY_ALLOCATE));
    void *p;
    CK(dnnl_memory_map_data(src_m, &p));
    memcpy(p, src, sizeof(src));
    CK(dnnl_memory_unmap_data(src_m, p));
    CK(dnnl_memory_map_data(sc_m, &p));
    memcpy(p, scale, sizeof(scale));
    CK(dnnl_memory_unmap_data(sc_m, p));

    dnnl_exec_arg_t args[3] = {{DNNL_ARG_FROM, src_m}, {DNNL_ARG_TO, dst_m}, {DNNL_ARG_ATTR_SCALES | DNNL_ARG_DST, sc_m}};
    CK(dnnl_primitive_execute(prim, strm, 3, args));
    CK(dnnl_stream_wait(strm));
    CK(dnnl_memory_map_data(dst_m, &p));
    memcpy(got, p, sizeof(got));
    CK(dnnl_memory_unmap_data(dst_m, p));

    int bad = 0;
    for (int r = 0; r < R; ++r)
        for (int c = 0; c < C; ++c) {
            float d = src[r * C + c] * (1.f / scale[r]);
            d = d < -128.f ? -128.f : d > 127.f ? 127.f : d;
            if ((int)nearbyintf(d) != (int)got[r * C + c]) ++bad;
        }
    if (bad) {
        printf("MISMATCH in %d elements\n", bad);
        return 2;
    }
    printf("OK %s\n", impl);
    dnnl_primitive_destroy(prim);
    dnnl_primitive_desc_destroy(pd);
    dnnl_primitive_attr_destroy(attr);
    dnnl_memory_destroy(src_m);
    dnnl_memory_destroy(dst_m);
    dnnl_memory_destroy(sc_m);
    dnnl_memory_desc_destroy(src_md);
    dnnl_memory_desc_destroy(dst_md);
    dnnl_memory_desc_destroy(sc_md);
    dnnl_stream_destroy(strm);
    dnnl_engine_destroy(eng);
    return 0;
}
