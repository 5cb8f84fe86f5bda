// Drives hvasconcelos/mlxforge's own configuration parser (src/core/config.cpp, compiled beside
// this file by tests/test_config_reference.py) over cases read from standard input, one JSON
// object a line: {"config": {...}, "override": "<json text>" (optional)}.  For every case it
// prints one JSON line: the parsed fields, or {"error": "<what the parser threw>"}.  The order
// of calls is the reference's own (src/runtime/engine.cpp: from_json, then the rope-scaling
// override if one is given, then validate_rope_scaling).
#include <iostream>
#include <string>

#include "core/config.h"

int main() {
  std::string line;
  while (std::getline(std::cin, line)) {
    if (line.empty()) continue;
    nlohmann::json out;
    try {
      const nlohmann::json in = nlohmann::json::parse(line);
      mlxforge::ModelConfig c = mlxforge::ModelConfig::from_json(in.at("config"));
      if (in.contains("override")) mlxforge::apply_rope_scaling_override(c, in.at("override").get<std::string>());
      mlxforge::validate_rope_scaling(c);
      out["model_type"] = c.model_type;
      out["num_hidden_layers"] = c.n_layers;
      out["hidden_size"] = c.hidden;
      out["num_attention_heads"] = c.n_heads;
      out["num_key_value_heads"] = c.n_kv_heads;
      out["head_dim"] = c.head_dim;
      out["vocab_size"] = c.vocab;
      out["intermediate_size"] = c.intermediate_size;
      out["rope_theta"] = c.rope_theta;
      out["rms_norm_eps"] = c.rms_eps;
      out["max_position_embeddings"] = c.max_position_embeddings;
      out["tie_word_embeddings"] = c.tie_word_embeddings;
      out["bos_token_id"] = c.bos_token_id;
      out["eos_token_ids"] = c.eos_token_ids;
      if (c.rope_scaling) {
        out["rope_scaling"] = {{"rope_type", c.rope_scaling->rope_type},
                               {"factor", c.rope_scaling->factor},
                               {"low_freq_factor", c.rope_scaling->low_freq_factor},
                               {"high_freq_factor", c.rope_scaling->high_freq_factor},
                               {"original_max_position_embeddings", c.rope_scaling->original_max_position_embeddings}};
      } else {
        out["rope_scaling"] = nullptr;
      }
    } catch (const std::exception& e) {
      out = nlohmann::json{{"error", e.what()}};
    }
    std::cout << out.dump() << std::endl;
  }
  return 0;
}
