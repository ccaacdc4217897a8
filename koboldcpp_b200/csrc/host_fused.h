// host_fused.h -- what the architectures that are served from a folder of named tensors share on the host side: tensor names
// "l<i>.<leaf>" and "mlp.e<j>.<which>", uploaded tensors that land as a slice of a larger fused tensor (q over k over v, gate over
// up, experts stacked), and the table of rotation frequencies.
#pragma once
#include "host_model.h"

namespace b200 {
namespace host {

struct Part { const char *leaf; int64_t rows; };
inline int64_t part_offset(const Part *p, int n, const char *leaf, int64_t *total, int64_t *rows = nullptr) {
    int64_t off = 0, found = -1;
    for (int i = 0; i < n; i++) {
        if (!strcmp(p[i].leaf, leaf)) { found = off; if (rows) *rows = p[i].rows; }
        off += p[i].rows;
    }
    if (total) *total = off;
    return found;
}

// "l<i>.<leaf>" -> i, leaf
inline bool split_name(const char *name, int *il, const char **leaf) {
    if (name[0] != 'l' || name[1] < '0' || name[1] > '9') return false;
    char *end = nullptr;
    const long v = strtol(name + 1, &end, 10);
    if (!end || *end != '.') return false;
    *il = (int)v;
    *leaf = end + 1;
    return true;
}
// "mlp.e<j>.<which>" -> j, which
inline bool split_expert(const char *leaf, int *e, const char **which) {
    if (strncmp(leaf, "mlp.e", 5) != 0 || leaf[5] < '0' || leaf[5] > '9') return false;
    char *end = nullptr;
    const long v = strtol(leaf + 5, &end, 10);
    if (!end || *end != '.') return false;
    *e = (int)v;
    *which = end + 1;
    return true;
}

// `data` becomes bytes [off, off + bytes) of the tensor `fused` (created with the given shape at the first part)
inline int place_into(b200_llama *m, const std::string &fused, const char *part_name, int type, int64_t ne0, int64_t ne1, int64_t ne2, size_t off, size_t bytes, const void *data) {
    ggml_tensor *f = find_w(m, fused);
    if (!f) {
        m->weight_pool.emplace_back();
        f = &m->weight_pool.back();
        memset(f, 0, sizeof(*f));
        set_shape(f, type, ne0, ne1, ne2, 1);
        snprintf(f->name, sizeof(f->name), "%s", fused.c_str());
        if (!alloc_in_buft(m, m->buft, f, GGML_BACKEND_BUFFER_USAGE_WEIGHTS)) {
            m->weight_pool.pop_back();
            b200::set_error("b200_llama_set_tensor: out of device memory for %s (%zu bytes)", fused.c_str(), nbytes(f));
            return B200_ERR_NOMEM;
        }
        m->weights[fused] = f;
        m->weight_bytes += (int64_t)nbytes(f);
    }
    LL_REQUIRE(f->type == type, B200_ERR_INVALID, "b200_llama_set_tensor: %s: the parts of %s must have one type", part_name, fused.c_str());
    LL_REQUIRE(m->weights.find(part_name) == m->weights.end(), B200_ERR_INVALID, "b200_llama_set_tensor: duplicate tensor %s", part_name);
    LL_REQUIRE(off + bytes <= nbytes(f), B200_ERR_INVALID, "b200_llama_set_tensor: %s does not fit %s", part_name, fused.c_str());
    f->buffer->iface.set_tensor(f->buffer, f, data, off, bytes);
    m->weights[part_name] = f;  // marks the part as present
    return B200_OK;
}

// per-pair rotation frequencies base^(-2i/dims), in double, rounded once; BANDS rescales by wavelength: short ones are kept, long
// ones divided by the factor, the band between blended linearly in original / wavelength
inline void rope_freqs(const b200_layer_params &lp, std::vector<float> &f) {
    const int dims = lp.rope_dims;
    f.resize((size_t)(dims / 2));
    for (int i = 0; i < dims / 2; i++) {
        double fi = pow((double)lp.rope_base, -2.0 * i / dims);
        if (lp.rope_scaling == B200_ROPE_SCALING_BANDS) {
            const double orig = lp.yarn_original, wl = 2.0 * M_PI / fi;
            if (wl > orig / lp.band_low) fi /= lp.yarn_factor;
            else if (!(wl < orig / lp.band_high)) {
                const double s = (orig / wl - lp.band_low) / ((double)lp.band_high - lp.band_low);
                fi = (1.0 - s) * fi / lp.yarn_factor + s * fi;
            }
        }
        f[(size_t)i] = (float)fi;
    }
}

}  // namespace host
}  // namespace b200
