// hybrid_config.hpp — configuration of the hybrid decoder family ("Ratasun"): a stack of parallel-residual layers whose token mixer is
// one of latent attention (a compressed key/value cache), a gated delta rule with per-channel decay, or a Mamba-2 state-space layer, each
// beside a routed mixture-of-experts feed-forward, with an optional looped block that re-injects the embedding.  Every size and constant
// is read from the checkpoint folder's config.json; nothing here is specific to one checkpoint.
#pragma once
#include <cstdio>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "json_dom.hpp"

namespace oa {

enum HyMixer : int { HY_LATENT_ATTENTION = 0, HY_CHANNEL_DELTA = 1, HY_MAMBA2 = 2 };

struct HyMoe {
    bool present = false;
    int experts = 0, top = 0, groups = 1, keep = 1, ff = 0;
    float scale = 1.f;
};

struct HyLayer {
    int type = HY_LATENT_ATTENTION;
    // latent attention: heads x (dim unrotated + rot_dim rotated) query/key, vdim values, kv_rank latent; rotary on the first rot_dims of the rotated part
    // channel delta:    heads value heads of vdim, kv_heads query/key heads of dim, conv taps
    // mamba2:           heads x vdim inner channels, state N, groups of B/C, norm_groups, conv taps
    int heads = 0, kv_heads = 0, dim = 0, rot_dim = 0, vdim = 0, kv_rank = 0, rot_dims = 0, conv = 0, state = 0, groups = 1, norm_groups = 1;
    float rot_base = 10000.f, scale = 1.f;
    HyMoe moe;
};

struct HyRun { int layer = 0, pass = -1; bool first_of_pass = false; int cache_idx = -1, state_idx = -1; };   // one execution of a layer (a looped layer runs once per pass)

struct HybridConfig {
    std::string dir;                      // checkpoint folder (config.json [+ model.safetensors]; without the latter the weights are seeded)
    int width = 0, vocab = 0;
    float eps = 1e-6f, logit_scale = 1.f;
    std::vector<HyLayer> layers;
    int loop_start = 0, loop_stop = 0, loop_times = 0;    // times == 0: no looped block
    std::vector<HyRun> runs;
    int n_caches = 0, n_states = 0;

    static double num(const Json& o, const char* k, const char* where) {
        const Json* j = o.get(k);
        if (!j || j->t != Json::Num) throw std::runtime_error(std::string("config.json: ") + where + " needs a number '" + k + "'");
        return j->n;
    }
    static int integer(const Json& o, const char* k, const char* where) { return (int)std::llround(num(o, k, where)); }
    static const Json& obj(const Json& o, const char* k, const char* where) {
        const Json* j = o.get(k);
        if (!j || j->t != Json::Obj) throw std::runtime_error(std::string("config.json: ") + where + " needs an object '" + k + "'");
        return *j;
    }

    static std::string read_file(const std::string& path) {
        std::ifstream f(path, std::ios::binary);
        if (!f) throw std::runtime_error("cannot read " + path);
        std::stringstream ss; ss << f.rdbuf(); return ss.str();
    }
    // the "architecture" key of <dir>/config.json (empty if there is none): the model registry dispatches on it
    static std::string architecture_of(const std::string& dir) {
        Json j; std::string err;
        if (!parse_json(read_file(dir + "/config.json"), j, err)) throw std::runtime_error("config.json: " + err);
        return j.str("architecture");
    }

    static HybridConfig load(const std::string& dir) {
        Json j; std::string err;
        if (!parse_json(read_file(dir + "/config.json"), j, err)) throw std::runtime_error("config.json: " + err);
        HybridConfig c; c.dir = dir;
        c.width = integer(j, "width", "the model"); c.vocab = integer(j, "vocab", "the model");
        c.eps = (float)num(obj(j, "norm", "the model"), "eps", "norm");
        c.logit_scale = j.get("logit_scale") ? (float)num(j, "logit_scale", "the model") : 1.f;
        const Json* ls = j.get("layers");
        if (!ls || ls->t != Json::Arr || ls->a.empty()) throw std::runtime_error("config.json: 'layers' must be a non-empty list");
        for (const Json& lj : ls->a) {
            HyLayer l; const std::string type = lj.str("type");
            const Json& m = obj(lj, "mixer", "a layer");
            if (type == "latent_attention") {
                l.type = HY_LATENT_ATTENTION;
                l.heads = integer(m, "heads", type.c_str()); l.dim = integer(m, "dim", type.c_str()); l.rot_dim = integer(m, "rot_dim", type.c_str());
                l.vdim = integer(m, "vdim", type.c_str()); l.kv_rank = integer(m, "kv_rank", type.c_str()); l.scale = (float)num(m, "scale", type.c_str());
                const Json& r = obj(m, "rot", type.c_str());
                l.rot_base = (float)num(r, "base", "rot"); l.rot_dims = integer(r, "dims", "rot");
                if (l.rot_dims > l.rot_dim || (l.rot_dims & 1)) throw std::runtime_error("config.json: rot.dims must be even and <= rot_dim");
            } else if (type == "channel_delta") {
                l.type = HY_CHANNEL_DELTA;
                l.heads = integer(m, "heads", type.c_str()); l.kv_heads = integer(m, "kv_heads", type.c_str()); l.dim = integer(m, "dim", type.c_str());
                l.vdim = integer(m, "vdim", type.c_str()); l.conv = integer(m, "conv", type.c_str());
                if (l.kv_heads <= 0 || l.heads % l.kv_heads) throw std::runtime_error("config.json: kv_heads must divide heads");
            } else if (type == "mamba2") {
                l.type = HY_MAMBA2;
                l.heads = integer(m, "heads", type.c_str()); l.vdim = integer(m, "vdim", type.c_str()); l.state = integer(m, "state", type.c_str());
                l.groups = integer(m, "groups", type.c_str()); l.norm_groups = integer(m, "norm_groups", type.c_str()); l.conv = integer(m, "conv", type.c_str());
                if (l.groups <= 0 || l.heads % l.groups || l.norm_groups <= 0 || (l.heads * l.vdim) % l.norm_groups) throw std::runtime_error("config.json: groups must divide heads, norm_groups the inner size");
            } else throw std::runtime_error("config.json: unknown layer type '" + type + "'");
            if (l.heads <= 0 || l.vdim <= 0 || (l.type != HY_LATENT_ATTENTION && (l.conv < 1 || l.conv > 16))) throw std::runtime_error("config.json: bad mixer sizes");
            const Json* mj = lj.get("mlp");
            if (mj && mj->t == Json::Obj) {
                if (mj->str("kind") != "moe") throw std::runtime_error("config.json: unknown mlp kind '" + mj->str("kind") + "'");
                const Json& r = obj(*mj, "router", "mlp");
                l.moe.present = true; l.moe.ff = integer(obj(*mj, "expert", "mlp"), "ff", "expert");
                l.moe.experts = integer(r, "experts", "router"); l.moe.top = integer(r, "top", "router"); l.moe.scale = (float)num(r, "scale", "router");
                if (const Json* g = r.get("groups")) if (g->t == Json::Obj) { l.moe.groups = integer(*g, "count", "groups"); l.moe.keep = integer(*g, "keep", "groups"); }
                if (l.moe.groups <= 0 || l.moe.experts % l.moe.groups || l.moe.keep <= 0 || l.moe.keep > l.moe.groups || l.moe.top <= 0 ||
                    l.moe.top > l.moe.keep * (l.moe.experts / l.moe.groups) || l.moe.top > 32 || l.moe.experts > 1024)
                    throw std::runtime_error("config.json: bad router sizes");
            }
            c.layers.push_back(l);
        }
        const Json* lp = j.get("loop");
        if (lp && lp->t == Json::Obj) {
            c.loop_start = integer(*lp, "start", "loop"); c.loop_stop = integer(*lp, "stop", "loop"); c.loop_times = integer(*lp, "times", "loop");
            if (c.loop_start < 0 || c.loop_stop <= c.loop_start || c.loop_stop > (int)c.layers.size() || c.loop_times < 1) throw std::runtime_error("config.json: bad loop");
        }
        // expand the schedule of layer executions: each execution owns its cache (attention) or state (recurrent mixers)
        auto add = [&](int layer, int pass, bool first) {
            HyRun r; r.layer = layer; r.pass = pass; r.first_of_pass = first;
            if (c.layers[layer].type == HY_LATENT_ATTENTION) r.cache_idx = c.n_caches++; else r.state_idx = c.n_states++;
            c.runs.push_back(r);
        };
        for (int i = 0; i < (int)c.layers.size();) {
            if (c.loop_times > 0 && i == c.loop_start) {
                for (int t = 0; t < c.loop_times; ++t) for (int k = c.loop_start; k < c.loop_stop; ++k) add(k, t, k == c.loop_start);
                i = c.loop_stop;
            } else { add(i, -1, false); ++i; }
        }
        if (c.width <= 0 || c.vocab <= 0) throw std::runtime_error("config.json: bad width / vocab");
        return c;
    }
};

}  // namespace oa
