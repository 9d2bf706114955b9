// Reader of the reference's `.otter` text graphs (Tensor/Otter.cpp:14-70 tokens, :117- blocks; used by
// Net::load_otter, Tensor/Net.cpp:518-536). Grammar, as the reference's own files use it:
//
//     name: "free text"                 <- file-level key/value pairs, ignored
//     LayerType {                       <- one block per layer; the block name is the layer type
//         key: value                    <- value is a bare word or a "quoted string" (may contain spaces and commas)
//         Param { key: value ... }      <- nested blocks are flattened into the layer's options
//     }
//     # comment to end of line          $ ends the file early
//
// Every block becomes one LayerOption (string -> string) with "type" set, handed to Net::addLayer in file order.
#include <cctype>
#include <fstream>
#include <sstream>

#include "otter_api.hpp"

namespace otter {

namespace {

struct Token {
    enum Kind { Word, Colon, Open, Close, End } kind;
    std::string text;
};

class Lexer {
public:
    explicit Lexer(std::string text) : s_(std::move(text)) {}
    Token next() {
        for (;;) {
            while (i_ < s_.size() && std::isspace((unsigned char)s_[i_])) ++i_;
            if (i_ < s_.size() && s_[i_] == '#') {
                while (i_ < s_.size() && s_[i_] != '\n') ++i_;
                continue;
            }
            break;
        }
        if (i_ >= s_.size() || s_[i_] == '$') return {Token::End, ""};
        const char c = s_[i_];
        if (c == ':') { ++i_; return {Token::Colon, ":"}; }
        if (c == '{') { ++i_; return {Token::Open, "{"}; }
        if (c == '}') { ++i_; return {Token::Close, "}"}; }
        if (c == '"') {
            const size_t e = s_.find('"', i_ + 1);
            std::string t = s_.substr(i_ + 1, e == std::string::npos ? std::string::npos : e - i_ - 1);
            i_ = e == std::string::npos ? s_.size() : e + 1;
            return {Token::Word, t};
        }
        size_t b = i_;
        while (i_ < s_.size() && !std::isspace((unsigned char)s_[i_]) && s_[i_] != ':' && s_[i_] != '{' && s_[i_] != '}') ++i_;
        return {Token::Word, s_.substr(b, i_ - b)};
    }

private:
    std::string s_;
    size_t i_ = 0;
};

// parses the inside of a block (after '{') into opt; nested blocks are flattened
bool parse_block(Lexer& lx, LayerOption& opt, std::string& err) {
    for (;;) {
        Token t = lx.next();
        if (t.kind == Token::Close) return true;
        if (t.kind != Token::Word) { err = "expected a key or '}' inside a block"; return false; }
        Token u = lx.next();
        if (u.kind == Token::Open) {
            if (!parse_block(lx, opt, err)) return false;
        } else if (u.kind == Token::Colon) {
            Token v = lx.next();
            if (v.kind != Token::Word) { err = "expected a value after '" + t.text + ":'"; return false; }
            opt[t.text] = v.text;
        } else {
            err = "expected ':' or '{' after '" + t.text + "'";
            return false;
        }
    }
}

}  // namespace

int parse_otter_text(const std::string& text, std::vector<LayerOption>& layers, std::string& err) {
    Lexer lx(text);
    for (;;) {
        Token t = lx.next();
        if (t.kind == Token::End) return 0;
        if (t.kind != Token::Word) { err = "expected a layer type or a file-level key"; return -1; }
        Token u = lx.next();
        if (u.kind == Token::Colon) {  // file-level key: value
            if (lx.next().kind != Token::Word) { err = "expected a value after '" + t.text + ":'"; return -1; }
            continue;
        }
        if (u.kind != Token::Open) { err = "expected '{' after layer type '" + t.text + "'"; return -1; }
        LayerOption opt;
        if (!parse_block(lx, opt, err)) return -1;
        opt["type"] = t.text;
        layers.push_back(std::move(opt));
    }
}

int Net::load_otter(const char* model_structure, CompileMode mode) {
    std::ifstream f(model_structure);
    if (!f) { error_ = std::string("cannot open ") + model_structure; return -1; }
    std::stringstream ss;
    ss << f.rdbuf();
    std::vector<LayerOption> layers;
    std::string err;
    if (parse_otter_text(ss.str(), layers, err) != 0) { error_ = "otter syntax: " + err; return -1; }
    for (auto& l : layers) addLayer(l);
    return compile(mode);
}

}  // namespace otter
