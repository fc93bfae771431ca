/* Thin C entry point over the reference's own GGUF reader (gguf.c, compiled
 * from where it lies in the reference tree by oracle/Makefile; never copied
 * into this repository).  TEST INFRASTRUCTURE ONLY: lets the tests compare
 * what the library's reader sees in a file with what the reference sees. */
#include <stdint.h>
#include <string.h>
#include "gguf.h"

/* 0 = found.  offset = the tensor's first byte counted from the start of the file. */
int ref_gguf_probe(const char *path, const char *name, uint32_t *type, uint32_t *n_dims, uint64_t *dims4,
                   uint64_t *file_offset, uint64_t *nbytes, uint32_t *alignment, uint64_t *n_tensors) {
    gguf_file g;
    char err[256];
    if (gguf_open(&g, path, err, sizeof err) != 0) return -1;
    int rc = -2;
    const gguf_tensor *t = gguf_tensor_find(&g, name);
    if (t) {
        *type = t->ggml_type;
        *n_dims = t->n_dims;
        for (int d = 0; d < 4; d++) dims4[d] = d < (int)t->n_dims ? t->dims[d] : 1;
        *file_offset = (uint64_t)((const uint8_t *)t->data - (const uint8_t *)g.map);
        *nbytes = t->nbytes;
        rc = 0;
    }
    *alignment = g.alignment;
    *n_tensors = g.n_tensors;
    gguf_close(&g);
    return rc;
}
