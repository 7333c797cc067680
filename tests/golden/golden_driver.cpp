// Runs a tiny Llama through the reference's own CPU classes and prints the logits.
//
// This program only calls the public classes of Mourya05/StrataKV (TransformerBlock,
// RMSNorm, Linear, BlockPool, PageTable); it is linked against the reference's CPU
// library by tests/golden/make_golden.py.  The Generator class is not used: it hides
// logits, truncates weights to BF16 and runs one sequence only.
//
// usage: golden_driver <weights_dir> <layers> <hidden> <ffn> <heads> <kv_heads> <vocab> <token>...
// <weights_dir> holds one raw little-endian float32 file per tensor, named as in the checkpoint.
#include "stratakv/layers/linear.h"
#include "stratakv/layers/rmsnorm.h"
#include "stratakv/memory/block_pool.h"
#include "stratakv/memory/page_table.h"
#include "stratakv/models/transformer_block.h"

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

using namespace stratakv;

static std::vector<float> read_raw(const std::string& dir, const std::string& name, std::size_t count) {
    std::ifstream in(dir + "/" + name + ".f32", std::ios::binary);
    if (!in) throw std::runtime_error("cannot open " + name);
    std::vector<float> values(count);
    in.read(reinterpret_cast<char*>(values.data()), static_cast<std::streamsize>(count * sizeof(float)));
    if (static_cast<std::size_t>(in.gcount()) != count * sizeof(float)) throw std::runtime_error("short file " + name);
    return values;
}

// The checkpoint stores W as [out, in]; Linear holds the logical [in, out] matrix.
static void set_linear(layers::Linear& linear, const std::vector<float>& w_out_in) {
    const std::size_t in = linear.input_dim(), out = linear.output_dim();
    for (std::size_t o = 0; o < out; ++o)
        for (std::size_t i = 0; i < in; ++i) linear.weight()[i * out + o] = w_out_in[o * in + i];
}

static void set_norm(layers::RMSNorm& norm, const std::vector<float>& gamma) {
    for (std::size_t i = 0; i < gamma.size(); ++i) norm.gamma()[i] = gamma[i];
}

int main(int argc, char** argv) {
    if (argc < 9) { std::fprintf(stderr, "usage: see the header of this file\n"); return 2; }
    const std::string dir = argv[1];
    const std::size_t layers_n = std::strtoul(argv[2], nullptr, 10), hidden = std::strtoul(argv[3], nullptr, 10);
    const std::size_t ffn = std::strtoul(argv[4], nullptr, 10), heads = std::strtoul(argv[5], nullptr, 10);
    const std::size_t kv_heads = std::strtoul(argv[6], nullptr, 10), vocab = std::strtoul(argv[7], nullptr, 10);
    std::vector<int> tokens;
    for (int i = 8; i < argc; ++i) tokens.push_back(std::atoi(argv[i]));
    const std::size_t head_dim = hidden / heads, kv_dim = kv_heads * head_dim;
    const int total_blocks = 16, block_size = 16;

    std::vector<std::unique_ptr<models::TransformerBlock>> blocks;
    std::vector<std::unique_ptr<memory::BlockPool>> pools;
    std::vector<std::unique_ptr<memory::PageTable>> pages;
    for (std::size_t l = 0; l < layers_n; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        auto block = std::make_unique<models::TransformerBlock>(hidden, ffn, heads, kv_heads, total_blocks, block_size);
        set_norm(block->input_norm(), read_raw(dir, p + "input_layernorm.weight", hidden));
        set_norm(block->post_attention_norm(), read_raw(dir, p + "post_attention_layernorm.weight", hidden));
        set_linear(block->attention().query_projection(), read_raw(dir, p + "self_attn.q_proj.weight", hidden * hidden));
        set_linear(block->attention().key_projection(), read_raw(dir, p + "self_attn.k_proj.weight", kv_dim * hidden));
        set_linear(block->attention().value_projection(), read_raw(dir, p + "self_attn.v_proj.weight", kv_dim * hidden));
        set_linear(block->attention().output_projection(), read_raw(dir, p + "self_attn.o_proj.weight", hidden * hidden));
        set_linear(block->gate_projection(), read_raw(dir, p + "mlp.gate_proj.weight", ffn * hidden));
        set_linear(block->up_projection(), read_raw(dir, p + "mlp.up_proj.weight", ffn * hidden));
        set_linear(block->down_projection(), read_raw(dir, p + "mlp.down_proj.weight", hidden * ffn));
        blocks.push_back(std::move(block));
        pools.push_back(std::make_unique<memory::BlockPool>(total_blocks, block_size));
        pages.push_back(std::make_unique<memory::PageTable>());
        pages.back()->allocate_sequence(0, *pools.back());
    }
    const std::vector<float> embedding = read_raw(dir, "model.embed_tokens.weight", vocab * hidden);
    layers::RMSNorm final_norm(hidden);
    set_norm(final_norm, read_raw(dir, "model.norm.weight", hidden));
    layers::Linear head(hidden, vocab);
    set_linear(head, read_raw(dir, "lm_head.weight", vocab * hidden));

    Tensor x({tokens.size(), hidden});
    for (std::size_t t = 0; t < tokens.size(); ++t)
        for (std::size_t c = 0; c < hidden; ++c) x[t * hidden + c] = embedding[static_cast<std::size_t>(tokens[t]) * hidden + c];
    for (std::size_t l = 0; l < layers_n; ++l) x = blocks[l]->forward(x, 0, *pages[l], *pools[l], true);
    const Tensor logits = head.forward(final_norm.forward(x));
    for (std::size_t i = 0; i < tokens.size() * vocab; ++i) std::printf("%.9g\n", static_cast<double>(logits[i]));
    return 0;
}
