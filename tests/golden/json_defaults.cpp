// Prints how wlejon/brolm's JSON reader treats absent, null and present keys of a config.json
// (include/brolm/detail/json.h:88-119: a getter returns its default for an absent or null key).
#include "brolm/detail/json.h"

#include <cstdio>
#include <string>

int main() {
    namespace j = brolm::detail::json;
    const std::string doc = R"({"hidden_size": 96, "head_dim": null, "rms_norm_eps": 1e-5,
                                "tie_word_embeddings": false, "vocab_size": 512.0, "rope_theta": null})";
    const j::Value root = j::parse(doc);
    std::printf("hidden_size %d\n", (int)root.get_int("hidden_size", 2304));
    std::printf("head_dim %d\n", (int)root.get_int("head_dim", 256));
    std::printf("num_hidden_layers %d\n", (int)root.get_int("num_hidden_layers", 26));
    std::printf("vocab_size %d\n", (int)root.get_int("vocab_size", 256000));
    std::printf("rms_norm_eps %.9g\n", (double)root.get_float("rms_norm_eps", 1e-6f));
    std::printf("rope_theta %.9g\n", (double)root.get_float("rope_theta", 10000.0f));
    std::printf("tie_word_embeddings %d\n", root.get_bool("tie_word_embeddings", true) ? 1 : 0);
    return 0;
}
