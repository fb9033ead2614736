// qwen35 model files: configuration from the metadata, fail-closed checks of what this library can run, and the weight
// source that feeds an engine under construction from the mapped file (Config::from_gguf, src/model.rs:16-47;
// load_hadamard, :50-62; Model::load, src/cpu.rs:91-112; MtpHead::validate_layout / load, src/mtp.rs:48-101).
#include "it_engine.h"
#include "it_gguf.h"
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <set>
#include <thread>

namespace {

const char* layer_tensor_name(int t) {
    switch (t) {
        case IT_T_ATTN_NORM: return "attn_norm.weight"; case IT_T_POST_NORM: return "post_attention_norm.weight";
        case IT_T_FFN_GATE: return "ffn_gate.weight"; case IT_T_FFN_UP: return "ffn_up.weight"; case IT_T_FFN_DOWN: return "ffn_down.weight";
        case IT_T_QKV: return "attn_qkv.weight"; case IT_T_GATE: return "attn_gate.weight"; case IT_T_CONV: return "ssm_conv1d.weight";
        case IT_T_DT: return "ssm_dt.bias"; case IT_T_A: return "ssm_a"; case IT_T_BETA: return "ssm_beta.weight"; case IT_T_ALPHA: return "ssm_alpha.weight";
        case IT_T_SSM_NORM: return "ssm_norm.weight"; case IT_T_SSM_OUT: return "ssm_out.weight";
        case IT_T_Q: return "attn_q.weight"; case IT_T_K: return "attn_k.weight"; case IT_T_V: return "attn_v.weight"; case IT_T_O: return "attn_output.weight";
        case IT_T_Q_NORM: return "attn_q_norm.weight"; case IT_T_K_NORM: return "attn_k_norm.weight";
    }
    return nullptr;
}
const char* head_tensor_name(int t) {
    switch (t) {
        case IT_T_MTP_EH: return "nextn.eh_proj.weight"; case IT_T_MTP_Q: return "attn_q.weight"; case IT_T_MTP_K: return "attn_k.weight";
        case IT_T_MTP_V: return "attn_v.weight"; case IT_T_MTP_O: return "attn_output.weight"; case IT_T_MTP_GATE: return "ffn_gate.weight";
        case IT_T_MTP_UP: return "ffn_up.weight"; case IT_T_MTP_DOWN: return "ffn_down.weight";
        case IT_T_MTP_ENORM: return "nextn.enorm.weight"; case IT_T_MTP_HNORM: return "nextn.hnorm.weight"; case IT_T_MTP_ATTN_NORM: return "attn_norm.weight";
        case IT_T_MTP_POST_NORM: return "post_attention_norm.weight"; case IT_T_MTP_Q_NORM: return "attn_q_norm.weight"; case IT_T_MTP_K_NORM: return "attn_k_norm.weight";
        case IT_T_MTP_HEAD_NORM: return "nextn.shared_head_norm.weight";
    }
    return nullptr;
}

struct GgufModel {
    it_gguf trunk, sidecar;
    const it_gguf* head = nullptr;                  // the file that holds the NextN block (trunk or sidecar), or null
    it_model_config cfg;
    int head_il = -1;                               // block index of the NextN layer in `head`
    std::set<std::string> folded, inverse;          // prism.hadamard.weight_names / inverse_weight_names
    std::map<size_t, std::vector<float>> signs;     // explicit sign vectors by width
    std::string output_name;                        // "output.weight", or the embedding table when the head is tied
};

int to_i32(uint64_t v, const char* key, int32_t* out) {
    if (v > 0x7fffffffull) return it_fail(IT_EFORMAT, "gguf: %s = %llu is out of range", key, (unsigned long long)v);
    *out = (int32_t)v; return IT_OK;
}

// Metadata -> configuration, with the checks the reference makes on the transform (version 1, normalised
// Sylvester-Walsh-Hadamard, sign modes "none" / "explicit") and the one this library adds: block size 1024.
int read_config(const it_gguf& g, int ctx_len, GgufModel* m) {
    const it_gguf_value* arch = g.get("general.architecture");
    if (!arch || arch->type != GV_STR || arch->s != "qwen35") return it_fail(IT_EUNSUPPORTED, "gguf: expected the qwen35 architecture, got %s", arch && arch->type == GV_STR ? arch->s.c_str() : "none");
    it_model_config& c = m->cfg; memset(&c, 0, sizeof c);
    auto U = [&](const char* key, int32_t* out) { uint64_t v; IT_TRY(g.u(std::string("qwen35.") + key, &v)); return to_i32(v, key, out); };
    uint64_t blocks = 0, nextn = 0;
    IT_TRY(g.u("qwen35.block_count", &blocks));
    if (const it_gguf_value* v = g.get("qwen35.nextn_predict_layers")) if (!v->as_u64(&nextn)) return it_fail(IT_EFORMAT, "gguf: bad qwen35.nextn_predict_layers");
    if (nextn > blocks) return it_fail(IT_EFORMAT, "gguf: more NextN layers than blocks");
    IT_TRY(to_i32(blocks - nextn, "block_count", &c.n_layer));         // NextN blocks follow the trunk and are not part of it
    IT_TRY(U("embedding_length", &c.n_embd)); IT_TRY(U("feed_forward_length", &c.n_ff));
    IT_TRY(U("attention.head_count", &c.n_head)); IT_TRY(U("attention.head_count_kv", &c.n_head_kv)); IT_TRY(U("attention.key_length", &c.head_dim));
    IT_TRY(U("rope.dimension_count", &c.n_rot)); IT_TRY(g.f("qwen35.rope.freq_base", &c.rope_base)); IT_TRY(g.f("qwen35.attention.layer_norm_rms_epsilon", &c.eps));
    if (const it_gguf_value* s = g.get("qwen35.rope.dimension_sections")) {
        if (s->type != GV_ARR || s->ints.size() < 4) return it_fail(IT_EFORMAT, "gguf: qwen35.rope.dimension_sections must hold four integers");
        for (int i = 0; i < 4; i++) c.rope_sections[i] = (int32_t)s->ints[i];
    }
    IT_TRY(U("ssm.conv_kernel", &c.conv_k)); IT_TRY(U("ssm.state_size", &c.ssm_state)); IT_TRY(U("ssm.group_count", &c.ssm_groups));
    IT_TRY(U("ssm.time_step_rank", &c.ssm_vheads)); IT_TRY(U("ssm.inner_size", &c.ssm_inner));
    c.full_attn_interval = 4;
    if (g.get("qwen35.full_attention_interval")) IT_TRY(U("full_attention_interval", &c.full_attn_interval));
    const it_gguf_tensor* tok; IT_TRY(g.need("token_embd.weight", &tok));
    if (tok->dims.size() != 2 || tok->dims[0] != (uint64_t)c.n_embd) return it_fail(IT_EFORMAT, "gguf: token_embd.weight is not [n_embd, n_vocab]");
    IT_TRY(to_i32(tok->dims[1], "vocabulary size", &c.n_vocab));
    c.ctx_len = ctx_len;
    // the activation transform
    uint64_t v = 0;
    if (const it_gguf_value* x = g.get("prism.hadamard.version")) if (!x->as_u64(&v) || v != 1) return it_fail(IT_EUNSUPPORTED, "gguf: unsupported prism.hadamard.version (only 1)");
    if (const it_gguf_value* x = g.get("prism.hadamard.transform")) if (x->type != GV_STR || x->s != "normalized-sylvester-walsh-hadamard") return it_fail(IT_EUNSUPPORTED, "gguf: unsupported Hadamard transform %s", x->s.c_str());
    const it_gguf_value* bs = g.get("prism.hadamard.block_size");
    if (!bs || !bs->as_u64(&v)) return it_fail(IT_EUNSUPPORTED, "gguf: the model carries no prism.hadamard.block_size; this library runs Hadamard-folded ternary models only");
    if (v != 1024) return it_fail(IT_EUNSUPPORTED, "gguf: Hadamard block size %llu (only 1024)", (unsigned long long)v);
    for (const std::string& s : g.strings("prism.hadamard.weight_names")) m->folded.insert(s);
    for (const std::string& s : g.strings("prism.hadamard.inverse_weight_names")) m->inverse.insert(s);
    bool grouped = false;
    if (const it_gguf_value* x = g.get("prism.hadamard.gdn_v_grouped")) x->as_bool(&grouped);
    c.gdn_v_grouped = grouped ? 1 : 0;
    std::string mode = "none";
    if (const it_gguf_value* x = g.get("prism.hadamard.sign_mode")) if (x->type == GV_STR) mode = x->s;
    if (mode == "explicit") {
        const it_gguf_value* w = g.get("prism.hadamard.sign_widths"); const it_gguf_value* sv = g.get("prism.hadamard.sign_values");
        if (!w || !sv || w->type != GV_ARR || sv->type != GV_ARR || w->ints.size() != w->count || sv->ints.size() != sv->count) return it_fail(IT_EFORMAT, "gguf: explicit sign mode needs integer sign_widths and sign_values");
        size_t off = 0;
        for (int64_t wd : w->ints) {
            if (wd <= 0 || (size_t)wd > sv->ints.size() - off) return it_fail(IT_EFORMAT, "gguf: Hadamard sign length mismatch");
            std::vector<float> s((size_t)wd);
            for (size_t i = 0; i < (size_t)wd; i++) {
                const int64_t x = sv->ints[off + i];
                if (x != 1 && x != -1) return it_fail(IT_EFORMAT, "gguf: Hadamard sign value %lld is not +-1", (long long)x);
                s[i] = (float)x;
            }
            m->signs[(size_t)wd] = std::move(s); off += (size_t)wd;
        }
        if (off != sv->ints.size()) return it_fail(IT_EFORMAT, "gguf: Hadamard sign length mismatch");
    } else if (mode != "none") return it_fail(IT_EUNSUPPORTED, "gguf: unsupported sign_mode %s", mode.c_str());
    m->output_name = g.tensor("output.weight") ? "output.weight" : "token_embd.weight";
    return IT_OK;
}

int expect_dims(const it_gguf_tensor* t, uint64_t d0, uint64_t d1) {
    const bool ok = d1 == 0 ? (t->nelem == d0) : (t->dims.size() == 2 && t->dims[0] == d0 && t->dims[1] == d1);
    if (!ok) return it_fail(IT_EFORMAT, "gguf: tensor %s has an unexpected shape", t->name.c_str());
    return IT_OK;
}
int check_f32_like(const it_gguf& g, const std::string& name, uint64_t n, const std::set<std::string>& folded) {
    const it_gguf_tensor* t; IT_TRY(g.need(name, &t)); IT_TRY(expect_dims(t, n, 0));
    if (t->type != GG_F32 && t->type != GG_F16 && t->type != GG_BF16) return it_fail(IT_EUNSUPPORTED, "gguf: tensor %s is %s; expected F32, F16 or BF16", name.c_str(), it_gg_type_name(t->type));
    if (folded.count(name)) return it_fail(IT_EUNSUPPORTED, "gguf: tensor %s is Hadamard-folded; only ternary matrices may be", name.c_str());
    return IT_OK;
}
int check_ternary(const GgufModel& m, const std::string& name, uint64_t rows, uint64_t cols) {
    const it_gguf_tensor* t; IT_TRY(m.trunk.need(name, &t)); IT_TRY(expect_dims(t, cols, rows));
    if (t->type != GG_PQ2_0 && t->type != GG_PTQ1_0) return it_fail(IT_EUNSUPPORTED, "gguf: tensor %s is %s; the device path runs ternary (PQ2_0 / PTQ1_0) matrices", name.c_str(), it_gg_type_name(t->type));
    if (!m.folded.count(name)) return it_fail(IT_EUNSUPPORTED, "gguf: ternary matrix %s is not Hadamard-folded (prism.hadamard.weight_names)", name.c_str());
    return IT_OK;
}

// Everything the engine will ask for, checked before any device work.
int check_trunk(const GgufModel& m) {
    const it_model_config& c = m.cfg; const it_gguf& g = m.trunk;
    const uint64_t e = c.n_embd, ff = c.n_ff, hd = c.head_dim, kvd = (uint64_t)c.n_head_kv * hd, q = (uint64_t)c.n_head * hd;
    const uint64_t cd = it_cfg_conv_dim(c), inner = c.ssm_inner, nv = c.ssm_vheads;
    for (int il = 0; il < c.n_layer; il++) {
        auto N = [&](int t) { return "blk." + std::to_string(il) + "." + layer_tensor_name(t); };
        IT_TRY(check_f32_like(g, N(IT_T_ATTN_NORM), e, m.folded)); IT_TRY(check_f32_like(g, N(IT_T_POST_NORM), e, m.folded));
        IT_TRY(check_ternary(m, N(IT_T_FFN_GATE), ff, e)); IT_TRY(check_ternary(m, N(IT_T_FFN_UP), ff, e)); IT_TRY(check_ternary(m, N(IT_T_FFN_DOWN), e, ff));
        if (it_cfg_recurrent(c, il)) {
            IT_TRY(check_ternary(m, N(IT_T_QKV), cd, e)); IT_TRY(check_ternary(m, N(IT_T_GATE), inner, e)); IT_TRY(check_ternary(m, N(IT_T_SSM_OUT), e, inner));
            IT_TRY(check_f32_like(g, N(IT_T_CONV), cd * c.conv_k, m.folded)); IT_TRY(check_f32_like(g, N(IT_T_DT), nv, m.folded)); IT_TRY(check_f32_like(g, N(IT_T_A), nv, m.folded));
            IT_TRY(check_f32_like(g, N(IT_T_BETA), nv * e, m.folded)); IT_TRY(check_f32_like(g, N(IT_T_ALPHA), nv * e, m.folded)); IT_TRY(check_f32_like(g, N(IT_T_SSM_NORM), c.ssm_state, m.folded));
        } else {
            IT_TRY(check_ternary(m, N(IT_T_Q), 2 * q, e)); IT_TRY(check_ternary(m, N(IT_T_K), kvd, e)); IT_TRY(check_ternary(m, N(IT_T_V), kvd, e)); IT_TRY(check_ternary(m, N(IT_T_O), e, q));
            IT_TRY(check_f32_like(g, N(IT_T_Q_NORM), hd, m.folded)); IT_TRY(check_f32_like(g, N(IT_T_K_NORM), hd, m.folded));
        }
    }
    IT_TRY(check_f32_like(g, "output_norm.weight", e, m.folded));
    IT_TRY(check_ternary(m, m.output_name, c.n_vocab, e));
    const it_gguf_tensor* tok; IT_TRY(g.need("token_embd.weight", &tok));
    return IT_OK;
}

// The NextN block: one layer, int8-group matrices, f32 norms, an optional embedding table of its own, no LM head of its
// own and no folded tensor (the reference refuses the same, src/mtp.rs:48-72).
int check_head(GgufModel& m) {
    const it_gguf& g = *m.head; const it_model_config& c = m.cfg;
    uint64_t blocks = 0, nextn = 0;
    IT_TRY(g.u("qwen35.block_count", &blocks)); IT_TRY(g.u("qwen35.nextn_predict_layers", &nextn));
    if (nextn != 1) return it_fail(IT_EUNSUPPORTED, "gguf: only a single NextN block is supported (the file has %llu)", (unsigned long long)nextn);
    if (blocks != (uint64_t)c.n_layer + 1) return it_fail(IT_EFORMAT, "gguf: the NextN head belongs to a trunk of %llu layers, not %d", (unsigned long long)(blocks - 1), c.n_layer);
    m.head_il = (int)blocks - 1;
    const std::string pre = "blk." + std::to_string(m.head_il) + ".";
    const uint64_t e = c.n_embd, q = (uint64_t)c.n_head * c.head_dim, kvd = (uint64_t)c.n_head_kv * c.head_dim, ff = c.n_ff;
    const struct { int t; uint64_t cols, rows; } mats[] = { { IT_T_MTP_EH, 2 * e, e }, { IT_T_MTP_Q, e, 2 * q }, { IT_T_MTP_K, e, kvd }, { IT_T_MTP_V, e, kvd },
        { IT_T_MTP_O, q, e }, { IT_T_MTP_GATE, e, ff }, { IT_T_MTP_UP, e, ff }, { IT_T_MTP_DOWN, ff, e } };
    for (const auto& x : mats) {
        const it_gguf_tensor* t; IT_TRY(g.need(pre + head_tensor_name(x.t), &t)); IT_TRY(expect_dims(t, x.cols, x.rows));
        if (t->type != GG_Q8_0 && t->type != GG_Q6_K) return it_fail(IT_EUNSUPPORTED, "gguf: unsupported NextN matrix type %s for %s (Q8_0 or Q6_K)", it_gg_type_name(t->type), t->name.c_str());
        if (x.rows % 4 || x.cols % 256) return it_fail(IT_EUNSUPPORTED, "gguf: unsupported NextN matrix shape for %s", t->name.c_str());
    }
    const std::set<std::string> none;
    for (int t = IT_T_MTP_ENORM; t <= IT_T_MTP_K_NORM; t++) {
        const uint64_t n = (t == IT_T_MTP_Q_NORM || t == IT_T_MTP_K_NORM) ? c.head_dim : e;
        IT_TRY(check_f32_like(g, pre + head_tensor_name(t), n, none));
        const it_gguf_tensor* x = g.tensor(pre + head_tensor_name(t));
        if (x->type != GG_F32) return it_fail(IT_EUNSUPPORTED, "gguf: NextN norm %s must be F32", x->name.c_str());
        const float* f = (const float*)g.data(*x);
        for (uint64_t i = 0; i < n; i++) { float v; memcpy(&v, f + i, 4); if (!std::isfinite(v)) return it_fail(IT_EFORMAT, "gguf: non-finite NextN norm %s", x->name.c_str()); }
    }
    if (g.tensor(pre + "nextn.shared_head_norm.weight")) IT_TRY(check_f32_like(g, pre + "nextn.shared_head_norm.weight", e, none));
    else if (!g.tensor("output_norm.weight") && !m.trunk.tensor("output_norm.weight")) return it_fail(IT_EFORMAT, "gguf: the NextN head has no head norm");
    if (const it_gguf_tensor* t = g.tensor(pre + "nextn.embed_tokens.weight")) {
        IT_TRY(expect_dims(t, e, c.n_vocab));
        size_t be, bb; if (!it_gg_block(t->type, &be, &bb)) return it_fail(IT_EUNSUPPORTED, "gguf: unsupported NextN embedding type %u", t->type);
    }
    if (g.tensor(pre + "nextn.shared_head_head.weight")) return it_fail(IT_EUNSUPPORTED, "gguf: a separate NextN LM head is not supported");
    for (const char* key : { "prism.hadamard.weight_names", "prism.hadamard.inverse_weight_names" })
        for (const std::string& s : g.strings(key)) if (s.compare(0, pre.size(), pre) == 0) return it_fail(IT_EUNSUPPORTED, "gguf: a Hadamard-folded NextN head is not supported");
    return IT_OK;
}

// A sidecar head must describe the same model: architecture, every qwen35.*, tokenizer.* and prism.hadamard.* key equal
// byte for byte, except the two block counts (validate_compatibility, src/mtp.rs:31-43).
int check_sidecar(const it_gguf& head, const it_gguf& trunk) {
    auto relevant = [](const std::string& k) {
        if (k == "qwen35.block_count" || k == "qwen35.nextn_predict_layers") return false;
        return k == "general.architecture" || k.compare(0, 7, "qwen35.") == 0 || k.compare(0, 10, "tokenizer.") == 0 || k.compare(0, 15, "prism.hadamard.") == 0;
    };
    for (int pass = 0; pass < 2; pass++) {
        const it_gguf& a = pass ? trunk : head; const it_gguf& b = pass ? head : trunk;
        for (const auto& kv : a.kv()) {
            if (!relevant(kv.first)) continue;
            const it_gguf_value* o = b.get(kv.first);
            if (!o || o->raw_len != kv.second.raw_len || memcmp(a.raw(kv.second), b.raw(*o), o->raw_len) != 0) return it_fail(IT_EFORMAT, "gguf: NextN head and trunk metadata differ: %s", kv.first.c_str());
        }
    }
    return IT_OK;
}

int open_model(const char* path, const char* head_path, int ctx_len, GgufModel* m) {
    IT_TRY(m->trunk.open(path));
    IT_TRY(read_config(m->trunk, ctx_len, m));
    IT_TRY(it_engine_validate_config(&m->cfg));
    IT_TRY(check_trunk(*m));
    if (head_path && *head_path && std::string(head_path) != path) {
        IT_TRY(m->sidecar.open(head_path));
        IT_TRY(check_sidecar(m->sidecar, m->trunk));
        m->head = &m->sidecar;
    } else if (head_path) {
        uint64_t nextn = 0;
        if (const it_gguf_value* v = m->trunk.get("qwen35.nextn_predict_layers")) v->as_u64(&nextn);
        if (nextn == 0) return it_fail(IT_EFORMAT, "gguf: %s holds no NextN block", path);
        m->head = &m->trunk;
    }
    if (m->head) IT_TRY(check_head(*m));
    return IT_OK;
}

// In-place normalised Walsh-Hadamard transform of each 1024-block, then the sign multiply: the inverse transform that
// brings a latent embedding row back to model space (Hadamard::inverse, src/hadamard.rs:44-49; butterflies in the
// order of fwht_blocks, :7-20, so every float comes out the same).
void inverse_hadamard_row(float* x, size_t n, const std::vector<float>* signs) {
    const float scale = 1.0f / sqrtf(1024.0f);
    for (size_t b = 0; b < n; b += 1024) {
        float* c = x + b;
        for (size_t h = 1; h < 1024; h *= 2)
            for (size_t i = 0; i < 1024; i += 2 * h)
                for (size_t j = i; j < i + h; j++) { const float p = c[j], q = c[j + h]; c[j] = p + q; c[j + h] = p - q; }
        for (size_t j = 0; j < 1024; j++) c[j] *= scale;
    }
    if (signs) for (size_t j = 0; j < n; j++) x[j] *= (*signs)[j];
}

struct GgufSource : it_weight_source {
    GgufModel* m;
    explicit GgufSource(GgufModel* model) : m(model) {}

    std::string name_of(int layer, int tensor) const {
        if (layer >= 0) return "blk." + std::to_string(layer) + "." + layer_tensor_name(tensor);
        if (tensor == IT_T_OUTPUT_NORM) return "output_norm.weight";
        if (tensor == IT_T_OUTPUT) return m->output_name;
        return "blk." + std::to_string(m->head_il) + "." + head_tensor_name(tensor);
    }
    int signs(it_engine*, size_t width, std::vector<float>* s) override {
        auto it = m->signs.find(width);
        if (it != m->signs.end()) *s = it->second; else s->assign(width, 1.0f);   // no vector for a width: no sign multiply
        return IT_OK;
    }
    // an embedding table: rows decoded on host threads, a slab of rows at a time, and copied up
    int table(it_engine* e, const it_gguf& g, const it_gguf_tensor* t, bool inverse, float* dev) {
        const size_t cols = (size_t)t->dims[0], rows = (size_t)t->dims[1];
        size_t be, bb; it_gg_block(t->type, &be, &bb);
        const size_t row_bytes = cols / be * bb;
        const std::vector<float>* sg = nullptr;
        if (inverse) { auto it = m->signs.find(cols); if (it != m->signs.end()) sg = &it->second; }
        const size_t slab = std::max<size_t>(1, std::min(rows, (size_t)(64u << 20) / (cols * 4)));
        std::vector<float> buf(slab * cols);
        const unsigned nthreads = std::max(1u, std::min(16u, std::thread::hardware_concurrency()));
        const uint8_t* src = g.data(*t);
        for (size_t r0 = 0; r0 < rows; r0 += slab) {
            const size_t nr = std::min(slab, rows - r0);
            std::vector<std::thread> pool;
            for (unsigned th = 0; th < nthreads; th++) pool.emplace_back([&, th]() {
                for (size_t r = th; r < nr; r += nthreads) {
                    float* row = buf.data() + r * cols;
                    it_gg_dequant(t->type, src + (r0 + r) * row_bytes, cols, row);
                    if (inverse) inverse_hadamard_row(row, cols, sg);
                }
            });
            for (std::thread& th : pool) th.join();
            IT_CUDA(cudaMemcpyAsync(dev + r0 * cols, buf.data(), nr * cols * 4, cudaMemcpyHostToDevice, e->ctx->stream));
            IT_CUDA(cudaStreamSynchronize(e->ctx->stream));
        }
        return IT_OK;
    }
    int f32(it_engine* e, int layer, int tensor, size_t n, float* dev) override {
        if (layer < 0 && tensor == IT_T_TOK_EMBD) {
            const it_gguf_tensor* t; IT_TRY(m->trunk.need("token_embd.weight", &t));
            return table(e, m->trunk, t, m->inverse.count("token_embd.weight") != 0, dev);
        }
        const it_gguf* g = &m->trunk;
        std::string name = name_of(layer, tensor);
        if (layer < 0 && tensor >= IT_T_MTP_ENORM) {
            g = m->head;
            if (tensor == IT_T_MTP_HEAD_NORM && !g->tensor(name)) { name = "output_norm.weight"; if (!g->tensor(name)) g = &m->trunk; }
        }
        const it_gguf_tensor* t; IT_TRY(g->need(name, &t));
        if (t->nelem != n) return it_fail(IT_EFORMAT, "gguf: tensor %s has %llu elements, expected %zu", name.c_str(), (unsigned long long)t->nelem, n);
        std::vector<float> host(n);
        IT_TRY(it_gg_dequant(t->type, g->data(*t), n, host.data()));
        IT_CUDA(cudaMemcpyAsync(dev, host.data(), n * 4, cudaMemcpyHostToDevice, e->ctx->stream));
        IT_CUDA(cudaStreamSynchronize(e->ctx->stream));
        return IT_OK;
    }
    int ternary(it_engine* e, int layer, int tensor, size_t rows, size_t cols, size_t row0, size_t nrows, uint8_t* raw_dev) override {
        const std::string name = name_of(layer, tensor);
        const it_gguf_tensor* t; IT_TRY(m->trunk.need(name, &t)); IT_TRY(expect_dims(t, cols, rows));
        const size_t nblk = nrows * (cols / 128);
        const uint8_t* src = m->trunk.data(*t);
        if (t->type == GG_PQ2_0) {
            IT_CUDA(cudaMemcpyAsync(raw_dev, src + row0 * (cols / 128) * 34, nblk * 34, cudaMemcpyHostToDevice, e->ctx->stream));
        } else if (t->type == GG_PTQ1_0) {
            std::vector<uint8_t> pq(nblk * 34);
            it_gg_ptq1_to_pq2(src + row0 * (cols / 128) * 28, nblk, pq.data());
            IT_CUDA(cudaMemcpyAsync(raw_dev, pq.data(), pq.size(), cudaMemcpyHostToDevice, e->ctx->stream));
        } else return it_fail(IT_EUNSUPPORTED, "gguf: tensor %s is not ternary", name.c_str());
        IT_CUDA(cudaStreamSynchronize(e->ctx->stream));
        return IT_OK;
    }
    int q8(it_engine* e, int tensor, size_t rows, size_t cols, it_qmat** out) override {
        const std::string name = name_of(-1, tensor);
        const it_gguf_tensor* t; IT_TRY(m->head->need(name, &t)); IT_TRY(expect_dims(t, cols, rows));
        const uint8_t* raw = m->head->data(*t);
        const bool k6 = t->type == GG_Q6_K;
        if (!k6 && t->type != GG_Q8_0) return it_fail(IT_EUNSUPPORTED, "gguf: NextN matrix %s is neither Q8_0 nor Q6_K", name.c_str());
        const size_t nblk = rows * cols / (k6 ? 256 : 32), stride = k6 ? 210 : 34, at = k6 ? 208 : 0;
        for (size_t i = 0; i < nblk; i++) {               // the reference refuses non-finite scales (src/mtp.rs:93)
            const unsigned short b = (unsigned short)(raw[i * stride + at] | (raw[i * stride + at + 1] << 8));
            if ((b & 0x7c00) == 0x7c00) return it_fail(IT_EFORMAT, "gguf: non-finite scale in NextN matrix %s", name.c_str());
        }
        return k6 ? it_qmatrix_upload_q6_k(e->ctx, raw, rows, cols, out) : it_qmatrix_upload_q8_0(e->ctx, raw, rows, cols, out);
    }
    int mtp_embd(it_engine* e, float** dev) override {
        const it_gguf_tensor* t = m->head->tensor("blk." + std::to_string(m->head_il) + ".nextn.embed_tokens.weight");
        if (!t) return IT_OK;
        float* p = nullptr;
        IT_TRY(it_engine_dev_alloc(e, (void**)&p, (size_t)t->nelem * 4, false));
        IT_TRY(table(e, *m->head, t, false, p));       // the head's own table is plain, not latent (src/mtp.rs:101)
        *dev = p; return IT_OK;
    }
};

}  // namespace

IT_API int it_gguf_inspect(const char* path, const char* head_path, int ctx_len, it_model_config* cfg, int* has_mtp, uint64_t* n_tensors, uint64_t* tensor_bytes) {
    IT_CHECK_ARG(path && cfg, "it_gguf_inspect: null argument");
    GgufModel m;
    IT_TRY(open_model(path, head_path, ctx_len, &m));
    *cfg = m.cfg;
    if (has_mtp) *has_mtp = m.head ? 1 : 0;
    if (n_tensors) *n_tensors = m.trunk.tensors().size();
    if (tensor_bytes) { uint64_t b = 0; for (const it_gguf_tensor& t : m.trunk.tensors()) b += t.nbytes; *tensor_bytes = b; }
    return IT_OK;
}

IT_API int it_engine_create_gguf(int device, const char* path, const char* head_path, int ctx_len, int rank, int world, it_engine** out) {
    IT_CHECK_ARG(path && out, "it_engine_create_gguf: null argument");
    *out = nullptr;
    GgufModel m;
    IT_TRY(open_model(path, head_path, ctx_len, &m));
    GgufSource src(&m);
    return it_engine_build(device, &m.cfg, 0, m.head ? 1 : 0, rank, world, &src, out);
}

IT_API int it_gguf_dequant(uint32_t ggml_type, const void* src, size_t n, float* out) {
    IT_CHECK_ARG(src && out, "it_gguf_dequant: null argument");
    return it_gg_dequant(ggml_type, (const uint8_t*)src, n, out);
}
IT_API int it_gguf_ptq1_to_pq2(const void* src, size_t nblocks, void* dst) {
    IT_CHECK_ARG(src && dst, "it_gguf_ptq1_to_pq2: null argument");
    it_gg_ptq1_to_pq2((const uint8_t*)src, nblocks, (uint8_t*)dst); return IT_OK;
}
