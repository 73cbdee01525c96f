/*
 * A host that is neither Python nor PyTorch: plain C against include/autograph_b200.h.
 *
 * It runs the call sequence that the reference's derived Forward makes for LeNet5
 * (benches/neural-network-benches/src/autograph_backend.rs:129-146: conv1 -> relu -> pool ->
 * conv2 -> relu -> pool -> flatten -> dense1 -> relu -> dense2 -> relu -> dense3) layer by layer
 * through the operator entry points, with every buffer coming from ag_alloc / ag_upload /
 * ag_download, and then the same network through ag_model_* (one kernel).  It reads
 *     <in>:  int32 batch, then f32 images [batch,1,28,28], then the six parameter tensors
 *            (conv1 [6,1,5,5], conv2 [16,6,5,5], dense1 [256,128], dense2 [128,84],
 *             dense3 [84,10], bias3 [10])
 * and writes to <out>: f32 logits [batch,10] of the layer-by-layer pass, then of the model pass.
 * Exit status 0 on success; the first failing call prints ag_last_error().
 *
 * Build: gcc -std=c11 -O2 -I include tests/c_driver/lenet5_forward.c \
 *            -L autograph_b200 -lautograph_b200 -Wl,-rpath,$PWD/autograph_b200 -o lenet5_forward
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "autograph_b200.h"

#define CHECK(call)                                                                   \
    do {                                                                              \
        int s_ = (call);                                                              \
        if (s_ != AG_OK) {                                                            \
            fprintf(stderr, "%s -> %d: %s\n", #call, s_, ag_last_error());            \
            return 1;                                                                 \
        }                                                                             \
    } while (0)

static int read_f32(FILE *f, float *dst, size_t n) { return fread(dst, sizeof(float), n, f) == n ? 0 : 1; }

int main(int argc, char **argv) {
    if (argc != 3) {
        fprintf(stderr, "usage: %s <input file> <output file>\n", argv[0]);
        return 2;
    }
    FILE *in = fopen(argv[1], "rb");
    if (!in) return 2;
    int32_t bs = 0;
    if (fread(&bs, sizeof bs, 1, in) != 1 || bs <= 0) return 2;
    const size_t lens[6] = {150, 2400, 256 * 128, 128 * 84, 84 * 10, 10};
    const size_t n_x = (size_t)bs * 784;
    float *x = malloc(n_x * sizeof(float));
    float *params[6];
    if (!x || read_f32(in, x, n_x)) return 2;
    for (int i = 0; i < 6; ++i) {
        params[i] = malloc(lens[i] * sizeof(float));
        if (!params[i] || read_f32(in, params[i], lens[i])) return 2;
    }
    fclose(in);

    ag_device *dev = NULL;
    CHECK(ag_device_create(0, &dev));

    /* ---- device buffers: the caller owns every one of them (Tensor::into_device) */
    void *d_x, *d_p[6], *d_c1, *d_p1, *d_c2, *d_p2, *d_h1, *d_h2, *d_y;
    CHECK(ag_alloc(dev, n_x * 4, &d_x));
    CHECK(ag_upload(dev, d_x, x, n_x * 4));
    for (int i = 0; i < 6; ++i) {
        CHECK(ag_alloc(dev, lens[i] * 4, &d_p[i]));
        CHECK(ag_upload(dev, d_p[i], params[i], lens[i] * 4));
    }
    CHECK(ag_alloc(dev, (size_t)bs * 6 * 24 * 24 * 4, &d_c1));
    CHECK(ag_alloc(dev, (size_t)bs * 6 * 12 * 12 * 4, &d_p1));
    CHECK(ag_alloc(dev, (size_t)bs * 16 * 8 * 8 * 4, &d_c2));
    CHECK(ag_alloc(dev, (size_t)bs * 16 * 4 * 4 * 4, &d_p2));
    CHECK(ag_alloc(dev, (size_t)bs * 128 * 4, &d_h1));
    CHECK(ag_alloc(dev, (size_t)bs * 84 * 4, &d_h2));
    CHECK(ag_alloc(dev, (size_t)bs * 10 * 4, &d_y));

    /* ---- the derived Forward, one call per layer */
    ag_conv2_options opt = {{5, 5}, {0, 0}, {1, 1}, {1, 1}};
    int64_t oh = 0, ow = 0;
    CHECK(ag_conv2_output_shape(28, 28, &opt, &oh, &ow));
    if (oh != 24 || ow != 24) return 3;
    CHECK(ag_conv2_forward(dev, AG_F32, d_x, bs, 1, 28, 28, d_p[0], 6, NULL, &opt, 0, d_c1));   /* conv1 */
    CHECK(ag_relu(dev, AG_F32, d_c1, d_c1, (int64_t)bs * 6 * 24 * 24));                           /* relu1 (relu_mut) */
    CHECK(ag_max_pool2(dev, AG_F32, d_c1, bs, 6, 24, 24, 2, 2, 2, 2, d_p1));                      /* pool1 */
    CHECK(ag_conv2_forward(dev, AG_F32, d_p1, bs, 6, 12, 12, d_p[1], 16, NULL, &opt, 0, d_c2));  /* conv2 */
    CHECK(ag_relu(dev, AG_F32, d_c2, d_c2, (int64_t)bs * 16 * 8 * 8));                            /* relu2 */
    CHECK(ag_max_pool2(dev, AG_F32, d_c2, bs, 16, 8, 8, 2, 2, 2, 2, d_p2));                       /* pool2 */
    /* flatten: [bs,16,4,4] is already [bs,256] in memory */
    CHECK(ag_gemm(dev, AG_F32, bs, 256, 128, 1.f, d_p2, 0, 256, 1, d_p[2], 0, 128, 1, 0.f, d_h1, 0, 128, 1)); /* dense1 = dot */
    CHECK(ag_relu(dev, AG_F32, d_h1, d_h1, (int64_t)bs * 128));                                   /* relu3 */
    CHECK(ag_gemm(dev, AG_F32, bs, 128, 84, 1.f, d_h1, 0, 128, 1, d_p[3], 0, 84, 1, 0.f, d_h2, 0, 84, 1));   /* dense2 */
    CHECK(ag_relu(dev, AG_F32, d_h2, d_h2, (int64_t)bs * 84));                                    /* relu4 */
    CHECK(ag_gemm(dev, AG_F32, bs, 84, 10, 1.f, d_h2, 0, 84, 1, d_p[4], 0, 10, 1, 0.f, d_y, 0, 10, 1));      /* dense3 */
    CHECK(ag_bias_add(dev, AG_F32, d_y, d_p[5], bs, 10, 1));                                      /* + bias */
    float *y1 = malloc((size_t)bs * 10 * sizeof(float));
    float *y2 = malloc((size_t)bs * 10 * sizeof(float));
    if (!y1 || !y2) return 2;
    CHECK(ag_download(dev, y1, d_y, (size_t)bs * 10 * 4));   /* into_array(): blocks */

    /* ---- the same network as a model object (LeNet5Classifier::infer) */
    ag_model *model = NULL;
    CHECK(ag_model_create_lenet5(dev, AG_F32, 1, &model));
    int32_t count = 0;
    CHECK(ag_model_parameter_count(model, &count));
    if (count != 6) return 3;
    for (int i = 0; i < 6; ++i) {
        int64_t len = 0;
        CHECK(ag_model_parameter_len(model, i, &len));
        if ((size_t)len != lens[i]) return 3;
        CHECK(ag_model_set_parameter(model, i, params[i]));
    }
    CHECK(ag_model_infer(model, x, bs, 1, 28, 28, y2));

    FILE *out = fopen(argv[2], "wb");
    if (!out) return 2;
    fwrite(y1, sizeof(float), (size_t)bs * 10, out);
    fwrite(y2, sizeof(float), (size_t)bs * 10, out);
    fclose(out);

    CHECK(ag_model_destroy(model));
    void *all[] = {d_x, d_c1, d_p1, d_c2, d_p2, d_h1, d_h2, d_y};
    for (size_t i = 0; i < sizeof all / sizeof all[0]; ++i) CHECK(ag_free(dev, all[i]));
    for (int i = 0; i < 6; ++i) CHECK(ag_free(dev, d_p[i]));
    CHECK(ag_device_wait(dev));
    CHECK(ag_device_destroy(dev));
    return 0;
}
