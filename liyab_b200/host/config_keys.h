// Readers of a configuration's keys that say what is wrong and where: every architecture's parser of config.json uses
// them, so that a missing or ill-typed key is reported in one form.
#pragma once

#include <cmath>
#include <format>
#include <string>

#include "json.h"
#include "spec.h"
#include "status.h"

namespace liyab {

inline int64_t int_in(const Json& obj, const char* key, const std::string& where, int64_t lo, int64_t hi = int64_t{1} << 30) {
    const Json* v = obj.find(key);
    if (v == nullptr || !v->is_int() || v->as_int() < lo || v->as_int() > hi)
        throw invalid_model("missing or invalid {}{} in config.json (got {}, need an integer in [{}, {}])", where, key, v == nullptr ? "nothing" : v->dump(), lo, hi);
    return v->as_int();
}

inline double number_in(const Json& obj, const char* key, const std::string& where) {
    const Json* v = obj.find(key);
    if (v == nullptr || !v->is_number() || !std::isfinite(v->as_number()))
        throw invalid_model("missing or invalid {}{} in config.json (got {}, need a finite number)", where, key, v == nullptr ? "nothing" : v->dump());
    return v->as_number();
}

inline const Json& object_in(const Json& obj, const char* key, const std::string& where) {
    const Json* v = obj.find(key);
    if (v == nullptr || !v->is_object()) throw invalid_model("missing or invalid {}{} in config.json (need an object)", where, key);
    return *v;
}

inline const Json* optional_in(const Json& obj, const char* key) {
    const Json* v = obj.find(key);
    return v == nullptr || v->is_null() ? nullptr : v;
}

// A parameter joined along its rows from several tensors of the file.
inline CheckpointTensor joined(std::vector<CheckpointSource> sources, ParamKind kind, double std_dev = 0.02, double mean = 0.0) {
    CheckpointTensor t;
    t.sources = std::move(sources);
    t.concat_axis = 0;
    t.kind = kind;
    t.init_mean = mean;
    t.init_std = std_dev;
    return t;
}


}  // namespace liyab
