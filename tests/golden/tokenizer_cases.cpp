// Prints what wlejon/brolm's own Gemma tokenizer (src/gemma_tokenizer.cpp with src/detail/spm_bpe.cpp and
// src/detail/byte_level_bpe.cpp, which build without the absent brotensor library) makes of the texts in
// tokenizer_cases.txt with the small tokenizer.json beside this file: one line of ids per text
// (tokenize, then encode with <bos> and <eos>), then the text decoded from the tokenize ids, in hex.
#include "brolm/gemma_tokenizer.h"

#include <cstdio>
#include <fstream>
#include <string>
#include <vector>

int main(int argc, char** argv) {
    if (argc < 3) return 2;
    auto tok = brolm::gemma::Tokenizer::load(argv[1]);
    std::printf("ids pad %d eos %d bos %d unk %d vocab %d\n", tok.pad_id(), tok.eos_id(), tok.bos_id(), tok.unk_id(),
                (int)tok.vocab_count());
    std::ifstream in(argv[2], std::ios::binary);
    std::string line;
    while (std::getline(in, line)) {
        // a line of the cases file is the text in hex (so that any bytes can be given)
        std::string text;
        for (std::size_t i = 0; i + 1 < line.size(); i += 2) text.push_back((char)std::stoi(line.substr(i, 2), nullptr, 16));
        const auto ids = tok.tokenize(text);
        std::printf("tokenize");
        for (int v : ids) std::printf(" %d", v);
        std::printf("\nencode");
        for (int v : tok.encode(text, true, true)) std::printf(" %d", v);
        std::printf("\ndecode ");
        for (unsigned char c : tok.decode(ids)) std::printf("%02x", c);
        std::printf("\n");
    }
    return 0;
}
