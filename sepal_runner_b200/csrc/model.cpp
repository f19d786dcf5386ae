#include "model.hpp"

#include <stdexcept>

namespace sepal::b200 {

namespace {

ModelGeometry preset(const char* name, std::uint64_t layers, std::uint64_t hidden, std::uint64_t mlp, std::uint64_t heads, std::uint64_t kv_heads,
                     std::uint64_t key_heads, std::uint64_t value_heads) {
    ModelGeometry g;
    g.name = name;
    g.layers = layers;
    g.hidden = hidden;
    g.intermediate = mlp;
    g.vocab = 248320;
    g.attn_heads = heads;
    g.attn_kv_heads = kv_heads;
    g.attn_head_dim = 256;
    g.dn_key_heads = key_heads;
    g.dn_value_heads = value_heads;
    g.dn_key_head_dim = 128;
    g.dn_value_head_dim = 128;
    g.conv_kernel = 4;
    g.attention_interval = 4;
    return g;
}

StorageProfile profile(const char* name, unsigned mlp, unsigned mixer, unsigned dn_out, unsigned dn_gates, unsigned small, unsigned group) {
    StorageProfile p;
    p.name = name;
    p.mlp = mlp;
    p.mixer = mixer;
    p.dn_out = dn_out;
    p.dn_gates = dn_gates;
    p.small = small;
    p.scale_group = group;
    return p;
}

}  // namespace

const std::vector<ModelGeometry>& model_presets() {
    static const std::vector<ModelGeometry> all = {
        preset("0.8b", 24, 1024, 3584, 8, 2, 16, 16),
        preset("2b", 24, 2048, 6144, 8, 2, 16, 16),
        preset("4b", 32, 2560, 9216, 16, 4, 16, 32),
        preset("9b", 32, 4096, 12288, 16, 4, 16, 32),
    };
    return all;
}

std::optional<ModelGeometry> find_model(std::string_view name) {
    for (const ModelGeometry& g : model_presets())
        if (g.name == name) return g;
    return std::nullopt;
}

const std::vector<StorageProfile>& storage_profiles() {
    static const std::vector<StorageProfile> all = {
        //       name        mlp mixer dn_out gates small group
        profile("w16",       2,  2,    2,     2,    2,    0),
        profile("w8",        1,  1,    1,     1,    1,    0),
        profile("gpu-f16",   2,  2,    2,     2,    4,    0),
        profile("gpu-q8w",   1,  1,    2,     2,    4,    0),
        profile("cpu-q8",    1,  1,    2,     2,    4,    0),
        profile("gpu-bf16",  2,  2,    2,     2,    4,    0),
        profile("gpu-w8g",   1,  2,    2,     2,    4,    128),  // the MLP alone is int8; the mixer projections stay 16-bit
    };
    return all;
}

std::optional<StorageProfile> find_profile(std::string_view name) {
    for (const StorageProfile& p : storage_profiles())
        if (p.name == name) return p;
    return std::nullopt;
}

ParameterCounts count_parameters(const ModelGeometry& g, unsigned scale_group, const StorageProfile* profile) {
    if (g.layers == 0 || g.hidden == 0 || g.attention_interval == 0 || g.layers % g.attention_interval != 0)
        throw std::invalid_argument("model geometry: the number of layers must be a positive multiple of the attention interval");
    const std::uint64_t h = g.hidden, n_attn = g.attention_layers(), n_dn = g.deltanet_layers();
    ParameterCounts n;
    n.mlp = g.layers * 3 * h * g.intermediate;                                           // gate, up [I, H]; down [H, I]
    n.small = g.layers * 2 * h + h;                                                      // two norms a layer, the final norm
    n.mixer = n_attn * (h * g.attn_in_width() + g.attn_width() * h);                     // [q + gate; k; v], o
    n.small += n_attn * 2 * g.attn_head_dim;                                             // q and k head norms
    n.mixer += n_dn * (h * g.dn_conv_dim() + h * g.dn_value_dim());                      // in_proj_qkv, in_proj_z
    n.dn_out = n_dn * g.dn_value_dim() * h;                                              // out_proj
    n.dn_gates = n_dn * 2 * h * g.dn_value_heads;                                        // in_proj_b, in_proj_a
    n.small += n_dn * (g.dn_conv_dim() * g.conv_kernel + 2 * g.dn_value_heads + g.dn_value_head_dim);  // conv, A_log, dt_bias, output norm
    if (scale_group != 0 && profile != nullptr) {
        const auto scales = [scale_group](std::uint64_t rows, std::uint64_t inputs) { return rows * ((inputs + scale_group - 1) / scale_group); };
        if (profile->mlp == 1) n.group_scales += g.layers * (2 * scales(g.intermediate, h) + scales(h, g.intermediate));
        if (profile->mixer == 1)
            n.group_scales += n_attn * (scales(g.attn_in_width(), h) + scales(h, g.attn_width())) + n_dn * (scales(g.dn_conv_dim(), h) + scales(g.dn_value_dim(), h));
        if (profile->dn_out == 1) n.group_scales += n_dn * scales(h, g.dn_value_dim());
        if (profile->dn_gates == 1) n.group_scales += n_dn * 2 * scales(g.dn_value_heads, h);
    }
    return n;
}

std::uint64_t trunk_weight_bytes(const ModelGeometry& g, const StorageProfile& p) {
    const ParameterCounts n = count_parameters(g, p.scale_group, &p);
    return n.mlp * p.mlp + n.mixer * p.mixer + n.dn_out * p.dn_out + n.dn_gates * p.dn_gates + n.small * p.small + n.group_scales * 4;
}

}  // namespace sepal::b200
