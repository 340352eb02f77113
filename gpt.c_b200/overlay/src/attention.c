/*
 * Host side of the Attention layer of gpt.c on top of libattn_sm100.so.
 *
 * Drop-in for src/attention.c of gpt.c: same constructor and struct of function pointers
 * (include/attention.h:42-61), same ownership rules, so src/self_attention.c, src/block.c,
 * src/transformer.c, train_gpt.c and infer_gpt.c compile and run against it unchanged.
 *
 * What differs from the reference layer (src/attention.c:54-157) on a CUDA device:
 *   - no q/k/v/att caches: nothing of size T x T is ever allocated.  The four cache slots hold
 *       cache[0]  the bf16 hi/lo split of the fused qkv tensor (what the kernels read)
 *       cache[1]  the log-sum-exp per (batch, head, token)            [B, H, T]
 *       cache[2]  a private copy of the layer output                  [B, T, C]
 *                 (the returned tensor is consumed and freed by the next Linear layer before
 *                  this layer's backward runs, src/linear.c:152,215)
 *       cache[3]  NULL
 *     all of them ordinary tensor_t, so free_cache / to / free_layer work as in the reference;
 *   - backward does not zero-fill its output (the kernels write every element).
 * On a CPU device the layer keeps the reference's cache layout and calls the reference's own CPU
 * kernel through the dispatch; the CUDA path has no CPU fallback.
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include "utils.h"
#include "dispatch.h"
#include "attention.h"
#include "attn_sm100.h"

static tensor_t *attn_forward(attention_t *attn, tensor_t *x);
static tensor_t *attn_backward(attention_t *attn, tensor_t *global_grad);
static void attn_description(const attention_t *attn);
static int attn_num_parameters(const attention_t *attn);
static void attn_free_layer(attention_t *attn);
static void attn_free_cache(attention_t *attn);
static void attn_to(attention_t *attn, const device_t device);

attention_t *Attention(int n_embd, int n_heads, int block_size) {
    CHECK_ERROR(n_heads <= 0 || n_embd % n_heads != 0,
                "Expected n_embd to be divisible by n_heads, but got n_embd = %d, n_heads = %d", n_embd, n_heads);
    attention_t *attn = (attention_t *)mallocCheck(sizeof(attention_t));

    /* The causal-mask buffer stays part of the public struct; only the CPU path reads it. */
    int mask_shape[2] = {block_size, block_size};
    attn->buffer = zeros(mask_shape, 2, CPU);
    for (int r = 0; r < block_size; r++) {
        float *line = attn->buffer->t + (size_t)r * block_size;
        for (int c = 0; c <= r; c++) line[c] = 1.0f;
    }
    for (int i = 0; i < 4; i++) attn->cache[i] = NULL;
    attn->n_embd = n_embd;
    attn->n_heads = n_heads;
    attn->forward = attn_forward;
    attn->backward = attn_backward;
    attn->description = attn_description;
    attn->num_parameters = attn_num_parameters;
    attn->free_layer = attn_free_layer;
    attn->free_cache = attn_free_cache;
    attn->to = attn_to;
    return attn;
}

/* A 1-D tensor_t big enough for `bytes` bytes (tensor_t counts floats). */
static tensor_t *byte_tensor(size_t bytes, device_t device) {
    CHECK_ERROR(bytes == 0 || bytes / sizeof(float) > 2147483647u, "attention: workspace of %zu bytes not representable", bytes);
    int shape[1] = {(int)((bytes + sizeof(float) - 1) / sizeof(float))};
    return create_tensor(shape, 1, device);
}

static tensor_t *attn_forward(attention_t *attn, tensor_t *x) {
    CHECK_ERROR(attn == NULL, "Expected *attn to be a attention_t pointer, but got NULL.");
    CHECK_ERROR(x == NULL, "Expected *x to be a tensor_t pointer, but got NULL.");
    CHECK_ERROR(x->ndims != 3 || x->shape[2] % 3 != 0, "Expected x of shape [B, T, 3C].");

    const int B = x->shape[0], T = x->shape[1], C = x->shape[2] / 3;
    const int H = attn->n_heads, D = C / H;
    const device_t device = x->device;

    int out_shape[3] = {B, T, C};
    tensor_t *out = create_tensor(out_shape, 3, device);
    attn_free_cache(attn); /* a forward without a backward in between (validation, inference) */

    if (device == CUDA) {
        int lse_shape[3] = {B, H, T};
        attn->cache[0] = byte_tensor(attn_sm100_saved_bytes(B, T, H, D), device);
        attn->cache[1] = create_tensor(lse_shape, 3, device);
        attn->cache[2] = create_tensor(out_shape, 3, device);
        attn->cache[3] = NULL;
    } else {
        int head_shape[4] = {B, H, T, D}, att_shape[4] = {B, H, T, T};
        attn->cache[0] = create_tensor(head_shape, 4, device);
        attn->cache[1] = create_tensor(head_shape, 4, device);
        attn->cache[2] = create_tensor(head_shape, 4, device);
        attn->cache[3] = create_tensor(att_shape, 4, device);
    }
    attention_forward_dispatch(x, attn->buffer, H, attn->cache, out);
    free_tensor(x); /* the layer consumes its input, as the reference does (src/attention.c:123) */
    return out;
}

static tensor_t *attn_backward(attention_t *attn, tensor_t *global_grad) {
    CHECK_ERROR(attn == NULL, "Expected *attn to be a attention_t pointer, but got NULL.");
    CHECK_ERROR(global_grad == NULL, "Expected *global_grad to be a tensor_t pointer, but got NULL.");
    CHECK_ERROR(attn->cache[0] == NULL, "attention backward called without a forward.");

    const int B = global_grad->shape[0], T = global_grad->shape[1], C = global_grad->shape[2];
    const device_t device = global_grad->device;
    int dx_shape[3] = {B, T, 3 * C};
    /* the CPU kernel assigns every element too (kernels/src/cpu/Attention.c:277-297) */
    tensor_t *dx = device == CUDA ? create_tensor(dx_shape, 3, device) : zeros(dx_shape, 3, device);

    attention_backward_dispatch(global_grad, attn->cache, attn->n_heads, dx);

    free_tensor(global_grad);
    attn_free_cache(attn);
    return dx;
}

static void attn_description(const attention_t *attn) {
    if (attn == NULL) return;
    printf("Attention(n_embd = %d, n_heads = %d)\n", attn->n_embd, attn->n_heads);
    printf("------------------------------------\n");
    printf("  n_embd : %d\n", attn->n_embd);
    printf("  n_heads: %d\n\n", attn->n_heads);
}

static int attn_num_parameters(const attention_t *attn) {
    (void)attn;
    return 0;
}

static void attn_free_cache(attention_t *attn) {
    if (attn == NULL) return;
    for (int i = 0; i < 4; i++) {
        free_tensor(attn->cache[i]); /* free_tensor(NULL) is a no-op */
        attn->cache[i] = NULL;
    }
}

static void attn_free_layer(attention_t *attn) {
    if (attn == NULL) return;
    free_tensor(attn->buffer);
    attn_free_cache(attn);
    free(attn);
}

static void attn_to(attention_t *attn, const device_t device) {
    CHECK_ERROR(attn == NULL, "Expected *attn to be a attention_t pointer, but got NULL.");
    attn->buffer->to(attn->buffer, device);
    for (int i = 0; i < 4; i++)
        if (attn->cache[i]) attn->cache[i]->to(attn->cache[i], device);
}
