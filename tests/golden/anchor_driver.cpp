// Runs the reference's own CPU Llama prefill graph on a model folder and writes the logits.
//
//   anchor <model folder> <tokens.txt (ids separated by blanks)> <out.f32>
//
// It only calls the reference's public functions, in the order its own test uses them
// (tests/test_smollm2_e2e.cpp:180-200): parse_config_json, load_safetensors,
// bind_smollm2_weights, build_forward_graph_prefill, Graph::build(CPU),
// populate_smollm2_weights, execute.  Output: [S, vocab] little-endian float32.
// Built by make_golden.py against the reference's source tree; no reference source is copied here.
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <iostream>
#include <span>
#include <sstream>
#include <string>
#include <vector>

#include "velomind/executable.h"
#include "velomind/graph.h"
#include "velomind/safetensors.h"
#include "velomind/tensor.h"
#include "llama_graph.h"
#include "model.h"
#include "model_loader.h"

int main(int argc, char** argv) {
    using namespace velomind;
    if (argc != 4) { std::cerr << "usage: anchor <folder> <tokens.txt> <out.f32>\n"; return 2; }
    const std::string folder = argv[1];
    std::ifstream cf(folder + "/config.json");
    std::stringstream cs; cs << cf.rdbuf();
    const auto cfg = examples::smollm2::parse_config_json(cs.str());
    auto sf = load_safetensors(folder + "/model.safetensors");
    if (!sf) { std::cerr << "cannot read model.safetensors\n"; return 1; }
    std::vector<std::int32_t> ids;
    { std::ifstream tf(argv[2]); std::int32_t t; while (tf >> t) ids.push_back(t); }
    const std::size_t S = ids.size();
    Graph g;
    auto tokens = g.input({static_cast<dim_t>(S)}, DataType::Int32);
    auto w = examples::smollm2::bind_smollm2_weights(g, cfg, S);
    auto logits = examples::llama::build_forward_graph_prefill(g, cfg, tokens, w);
    auto exec = g.build(DeviceType::CPU);
    if (!exec) { std::cerr << "graph build failed\n"; return 1; }
    examples::smollm2::populate_smollm2_weights(*sf, cfg, w, S);
    tokens.copy_from_host(std::as_bytes(std::span(ids)));
    exec->execute();
    std::vector<float> out(S * cfg.vocab_size);
    logits.copy_to_host(std::as_writable_bytes(std::span(out)));
    std::ofstream of(argv[3], std::ios::binary);
    of.write(reinterpret_cast<const char*>(out.data()), static_cast<std::streamsize>(out.size() * sizeof(float)));
    std::cout << "wrote " << S << " x " << cfg.vocab_size << " logits\n";
    return 0;
}
