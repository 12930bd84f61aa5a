// trace.cpp — Engine::replay_trace: feeds given token ids through the resident model step by step and writes the logits at the
// places a step asks for.  Nothing is sampled.  One JSON object per input line:
//     {"step": 3, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
// `tokens` are the request's NEXT tokens (the model continues from the cache the earlier steps left), `want` indexes into them,
// `end` lists requests whose cache rows are given back after the step.  For a step that wants something, <out_dir>/<step>.f32
// holds the logits [wanted, vocab] as little-endian F32 in entry / want order.  After every step "done <step>" is printed.
// The engine holds one sequence at a time (one flat cache): a request must end before another begins.
#include "engine.h"
#include "json.h"
#include <map>

namespace nt { namespace b200 {

namespace {
bool read_line(FILE* in, std::string& line) {
    line.clear();
    int c;
    while ((c = fgetc(in)) != EOF) { if (c == '\n') return true; line += (char)c; }
    return !line.empty();
}
}  // namespace

int Engine::replay_trace(FILE* in, const std::string& out_dir) {
    std::map<std::string, int> held;        // live request -> tokens in the cache
    const int vocab = model_.config().vocab_size;
    std::vector<float> logits;
    std::string line;
    while (read_line(in, line)) {
        if (line.find_first_not_of(" \t\r") == std::string::npos) continue;
        Json step;
        std::string err;
        if (!Json::parse(line, step, &err) || !step.is_object()) { fprintf(stderr, "trace: %s\n", err.c_str()); return 1; }
        const long long step_no = step.at("step").int_or(-1);
        std::vector<float> wanted_all;
        for (const Json& e : step.at("entries").arr) {
            const std::string id = e.at("id").is_string() ? e.at("id").str : std::to_string(e.at("id").int_or(0));
            std::vector<int> toks, want;
            for (const Json& t : e.at("tokens").arr) toks.push_back((int)t.int_or(-1));
            for (const Json& w : e.at("want").arr) want.push_back((int)w.int_or(-1));
            if (toks.empty()) continue;
            auto it = held.find(id);
            if (it == held.end()) {
                if (!held.empty()) {       // one flat cache: the newcomer takes it over
                    fprintf(stderr, "trace: request %s begins while %s is live; this engine holds one sequence at a time, the older one is dropped\n", id.c_str(), held.begin()->first.c_str());
                    held.clear();
                }
                it = held.emplace(id, 0).first;
            }
            const int start = it->second;
            if (start + (int)toks.size() > model_.config().max_seq_len) { fprintf(stderr, "trace: request %s outgrows the cache (%d tokens)\n", id.c_str(), model_.config().max_seq_len); return 1; }
            for (int t : toks) if (t < 0 || t >= vocab) { fprintf(stderr, "trace: token id out of range in request %s\n", id.c_str()); return 1; }
            logits.resize((size_t)want.size() * vocab);
            model_.forward_logits(toks.data(), (int)toks.size(), start, want.data(), (int)want.size(), logits.data());
            it->second += (int)toks.size();
            wanted_all.insert(wanted_all.end(), logits.begin(), logits.end());
        }
        for (const Json& e : step.at("end").arr) held.erase(e.is_string() ? e.str : std::to_string(e.int_or(0)));
        if (!wanted_all.empty()) {
            const std::string path = out_dir + "/" + std::to_string(step_no) + ".f32";
            FILE* f = fopen(path.c_str(), "wb");
            if (!f || fwrite(wanted_all.data(), sizeof(float), wanted_all.size(), f) != wanted_all.size()) { fprintf(stderr, "trace: cannot write %s\n", path.c_str()); if (f) fclose(f); return 1; }
            fclose(f);
        }
        printf("done %lld\n", step_no);
        fflush(stdout);
    }
    return 0;
}

}}  // namespace nt::b200
