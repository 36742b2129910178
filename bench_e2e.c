/* Host loop of bench.py's end-to-end leg, in C: what a C or C++ host of the plugin does per call --
 *   copy the call's activations from page-locked host memory to the device   (buffer_copy_from_host_async),
 *   the quantized matmul                                                      (qmatmul | qmatmul_sharded_push),
 *   read the result back into page-locked host memory, blocking               (buffer_copy_to_host)
 * -- through the plugin's own entry points, which bench.py hands over as function pointers taken from the
 * tables the plugin publishes.  Only the loop lives here (from Python every call costs about two microseconds
 * of interpreter and ctypes time that no such host pays); bench.py brackets it with the plugin's timers.
 * Built by __graft_entry__.build() with the host compiler; no CUDA, no plugin header needed. */
#include <stddef.h>
#include <stdint.h>

typedef int (*copy_in_fn)(void* ctx, void* buf, const void* src, size_t bytes);
typedef int (*copy_out_fn)(void* ctx, void* buf, void* dst, size_t bytes);
typedef int (*qmatmul_fn)(void* ctx, void* x, void* wq, void* scales, void* biases, void* y, int M, int K, int N, int bits,
                          int group, int x_dtype, int sb_dtype, int y_dtype);
typedef int (*push_fn)(void* y_symm, void* x, void* wq, void* scales, void* biases, int M, int K, int N_local, int bits,
                       int group, int y_dtype);

typedef struct {
    void *x_dev, *wq, *scales, *biases;
    void* y_dev;   /* the buffer read back (for a sharded call: the symmetric buffer seen as a buffer) */
    void* y_symm;  /* sharded calls: the symmetric buffer handle; else NULL */
    const void* x_host;
    void* y_host;
    size_t x_bytes, y_bytes;
    int32_t M, K, N, bits, group, dtype;
} lux_bench_call;

__attribute__((visibility("default")))
int lux_bench_e2e(copy_in_fn copy_in, qmatmul_fn qmatmul, push_fn push, copy_out_fn copy_out, void* ctx,
                  const lux_bench_call* calls, int n_calls, int reps, long long* calls_done) {
    long long done = 0;
    for (int r = 0; r < reps; r++) {
        for (int i = 0; i < n_calls; i++) {
            const lux_bench_call* c = &calls[i];
            int rc = copy_in(ctx, c->x_dev, c->x_host, c->x_bytes);
            if (rc) return rc;
            rc = c->y_symm ? push(c->y_symm, c->x_dev, c->wq, c->scales, c->biases, c->M, c->K, c->N, c->bits, c->group, c->dtype)
                           : qmatmul(ctx, c->x_dev, c->wq, c->scales, c->biases, c->y_dev, c->M, c->K, c->N, c->bits, c->group,
                                     c->dtype, c->dtype, c->dtype);
            if (rc) return rc;
            rc = copy_out(ctx, c->y_dev, c->y_host, c->y_bytes);
            if (rc) return rc;
            done++;
        }
    }
    if (calls_done) *calls_done = done;
    return 0;
}

/* The same for a whole sweep of independent matmuls handed to the plugin as ONE call (qmatmul_batch |
 * qmatmul_sharded_push_batch): the activations of all items lie one after another in one device buffer and
 * one page-locked host buffer (the items' x are views into it), and so do the outputs, so that a sweep is
 *   one host->device copy of every item's activations,
 *   one batched call,
 *   one blocking device->host copy of every item's output. */
typedef int (*batch_fn)(void* ctx, int n, void* const* x, void* const* wq, void* const* scales, void* const* biases,
                        void* const* y, const int* M, int K, int N, int bits, int group, int y_dtype);
typedef int (*push_batch_fn)(void* y_symm, int n, void* const* x, void* const* wq, void* const* scales, void* const* biases,
                             const size_t* y_offset, const int* M, int K, int N_local, int bits, int group, int y_dtype);

typedef struct {
    void* x_all_dev;
    const void* x_all_host;
    size_t x_bytes;
    void* y_all_dev; /* for a sharded call: the symmetric buffer seen as a buffer */
    void* y_all_host;
    size_t y_bytes;
    int32_t n;
    void* const* x;
    void* const* wq;
    void* const* scales;
    void* const* biases;
    void* const* y;         /* unsharded: the items' outputs, views into y_all_dev */
    const size_t* y_offset; /* sharded: the items' byte offsets inside the symmetric buffer */
    const int* M;
    void* y_symm; /* sharded: the symmetric buffer handle; else NULL */
    int32_t K, N, bits, group, dtype;
} lux_bench_batch;

__attribute__((visibility("default")))
int lux_bench_e2e_batch(copy_in_fn copy_in, batch_fn batch, push_batch_fn push_batch, copy_out_fn copy_out, void* ctx,
                        const lux_bench_batch* b, int reps, long long* matmuls_done) {
    long long done = 0;
    for (int r = 0; r < reps; r++) {
        int rc = copy_in(ctx, b->x_all_dev, b->x_all_host, b->x_bytes);
        if (rc) return rc;
        rc = b->y_symm ? push_batch(b->y_symm, b->n, b->x, b->wq, b->scales, b->biases, b->y_offset, b->M, b->K, b->N, b->bits,
                                    b->group, b->dtype)
                       : batch(ctx, b->n, b->x, b->wq, b->scales, b->biases, b->y, b->M, b->K, b->N, b->bits, b->group, b->dtype);
        if (rc) return rc;
        rc = copy_out(ctx, b->y_all_dev, b->y_all_host, b->y_bytes);
        if (rc) return rc;
        done += b->n;
    }
    if (matmuls_done) *matmuls_done = done;
    return 0;
}

/* Two sweeps in flight: the host keeps two contexts (two streams), each with its own activations and outputs,
 * and reads sweep r-1 back (blocking) while sweep r computes -- the copies of one context run under the kernels
 * of the other.  One GPU only: the batched sharded kernels of two contexts would wait for their peers from two
 * streams of one GPU.  Every sweep is still one copy in, one qmatmul_batch call, one blocking copy out. */
__attribute__((visibility("default")))
int lux_bench_e2e_batch2(copy_in_fn copy_in, batch_fn batch, copy_out_fn copy_out, void* const ctx[2],
                         const lux_bench_batch* const b[2], int reps, long long* matmuls_done) {
    long long done = 0;
    for (int r = 0; r <= reps; r++) {
        if (r < reps) {
            const lux_bench_batch* c = b[r & 1];
            int rc = copy_in(ctx[r & 1], c->x_all_dev, c->x_all_host, c->x_bytes);
            if (rc) return rc;
            rc = batch(ctx[r & 1], c->n, c->x, c->wq, c->scales, c->biases, c->y, c->M, c->K, c->N, c->bits, c->group, c->dtype);
            if (rc) return rc;
        }
        if (r > 0) {
            const lux_bench_batch* p = b[(r - 1) & 1];
            int rc = copy_out(ctx[(r - 1) & 1], p->y_all_dev, p->y_all_host, p->y_bytes);
            if (rc) return rc;
            done += p->n;
        }
    }
    if (matmuls_done) *matmuls_done = done;
    return 0;
}
