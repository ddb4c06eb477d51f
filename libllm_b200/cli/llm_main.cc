// The `llm` command line, in the manner of the reference's (go/bin/main.go:37-53):
//
//     llm chat -m FOLDER [-device auto|cuda] [-dtype bfloat16|float32]
//     llm generate -m FOLDER --prompt-ids 1,2,3 [--prompt-ids ...] [--max-new-tokens N]
//                  [--temperature T] [--top-k K] [--top-p P] [--seed S] [--no-stop] [--stop-ids a,b]
//
// `chat` is the reference's loop (go/bin/chat.go:67-131): a prompt per line, `:new` starts a new
// session, `:sys TEXT` sets what every session starts with, and after each reply a line with the
// number of tokens, the time and the milliseconds per token.  Text is not part of this library,
// so a line is a list of token ids (separated by spaces or commas) and the reply is printed as
// ids; a session keeps its history and every turn runs the whole history again, as the
// reference's chat does (go/bin/chat.go:107-112).  The sampler's defaults are the reference's:
// temperature 1.0, top_k 50, top_p 0.8 (src/libllm/llm.cc:125-132).  `generate` does not exist in
// the reference: it is the batched entry point on the command line, one prompt per
// `--prompt-ids`; each reply is one line of ids on standard output.  `download` is not built (no
// network; model folders are local).
//
// The program is a client of the C interface (include/llm.h), as the reference's is of its own
// (go/llm/llm.go:58-140).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "include/llm.h"

namespace {

struct Fail {
  std::string message;
};

void check(int32_t status) {
  if (status != LLM_OK) throw Fail{llm_get_last_error_message()};
}

// A JSON handle that frees itself.
struct JsonHandle {
  llm_json_t j = nullptr;
  JsonHandle() { check(llm_json_init(&j)); }
  explicit JsonHandle(const std::string &text) {
    check(llm_json_init(&j));
    check(llm_json_parse(&j, text.c_str()));
  }
  ~JsonHandle() { llm_json_destroy(&j); }
  std::string dump() {
    std::string buf((size_t)llm_json_dump_size(&j), '\0');
    check(llm_json_dump(&j, &buf[0], (int64_t)buf.size()));
    buf.resize(strlen(buf.c_str()));
    return buf;
  }
};

std::vector<long long> parse_ids(const std::string &text) {
  std::vector<long long> out;
  std::string cur;
  auto flush = [&] {
    if (cur.empty()) return;
    char *end = nullptr;
    const long long v = strtoll(cur.c_str(), &end, 10);
    if (*end) throw Fail{"'" + cur + "' is not a token id"};
    out.push_back(v);
    cur.clear();
  };
  for (char c : text) {
    if (c == ',' || c == ' ' || c == '\t' || c == '\n' || c == '\r') flush();
    else cur.push_back(c);
  }
  flush();
  return out;
}

std::string ids_json(const std::vector<long long> &ids) {
  std::string s = "[";
  for (size_t i = 0; i < ids.size(); ++i) s += (i ? "," : "") + std::to_string(ids[i]);
  return s + "]";
}

// Options: `-name value`, `--name value`, `--name=value`; flags without a value are listed in `flags`.
struct Args {
  std::map<std::string, std::vector<std::string>> values;
  bool has(const std::string &k) const { return values.count(k) != 0; }
  std::string get(const std::string &k, const std::string &fallback) const {
    auto it = values.find(k);
    return it == values.end() ? fallback : it->second.back();
  }
};

Args parse_args(int argc, char **argv, int first, const std::vector<std::string> &known, const std::vector<std::string> &flags,
                const std::map<std::string, std::string> &alias) {
  Args a;
  for (int i = first; i < argc; ++i) {
    std::string arg = argv[i];
    if (arg.size() < 2 || arg[0] != '-') throw Fail{"unexpected argument '" + arg + "'"};
    std::string name = arg.substr(arg[1] == '-' ? 2 : 1), value;
    bool has_value = false;
    const size_t eq = name.find('=');
    if (eq != std::string::npos) {
      value = name.substr(eq + 1);
      name = name.substr(0, eq);
      has_value = true;
    }
    for (auto &c : name)
      if (c == '_') c = '-';
    if (alias.count(name)) name = alias.at(name);
    bool is_flag = false, ok = false;
    for (const auto &f : flags) is_flag = is_flag || f == name;
    for (const auto &k : known) ok = ok || k == name;
    if (name == "h" || name == "help") {
      a.values["help"].push_back("1");
      continue;
    }
    if (!ok && !is_flag) throw Fail{"unknown option '" + arg + "'"};
    if (is_flag) {
      a.values[name].push_back("1");
      continue;
    }
    if (!has_value) {
      if (i + 1 >= argc) throw Fail{"option '" + arg + "' needs a value"};
      value = argv[++i];
    }
    a.values[name].push_back(value);
  }
  return a;
}

const std::vector<std::string> COMMON = {"model", "device", "dtype", "max-tokens", "max-seq-len"};
const std::map<std::string, std::string> ALIAS = {{"m", "model"}};

void usage() {
  fprintf(stderr,
          "Usage: llm COMMAND\n\nCommands:\n"
          "    chat           Chat with LLM (token ids in, token ids out)\n"
          "    generate       Generate continuations of one or more prompts\n\n"
          "Run 'llm COMMAND -h' for more information on a command.\n");
}

void common_help() {
  fprintf(stderr,
          "  -m, --model FOLDER       the model folder (config.json and model.safetensors)\n"
          "  -device auto|cuda        inference device (there is no cpu path)\n"
          "  -dtype bfloat16|float32  the engine's type (default bfloat16)\n"
          "  --max-tokens N           tokens the cache holds (default 65536)\n"
          "  --max-seq-len N          longest sequence (default: the model's)\n");
}

struct Model {
  llm_model_t m = nullptr;
  ~Model() { llm_model_destroy(&m); }
};

void load_model(const Args &a, Model *model) {
  if (!a.has("model")) throw Fail{"the option -m FOLDER is required"};
  const std::string device = a.get("device", "auto");
  std::string kw = "{\"filename\": \"";
  for (char c : a.get("model", "")) {
    if (c == '"' || c == '\\') kw.push_back('\\');
    kw.push_back(c);
  }
  kw += "\", \"device\": \"" + device + "\", \"dtype\": \"" + a.get("dtype", "bfloat16") + "\", \"max_tokens\": " +
        a.get("max-tokens", "65536");
  if (a.has("max-seq-len")) kw += ", \"max_seq_len\": " + a.get("max-seq-len", "0");
  kw += "}";
  JsonHandle kwargs(kw);
  check(llm_model_init(&model->m));
  check(llm_model_load(&model->m, &kwargs.j));
}

double now() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int chat_main(int argc, char **argv) {
  std::vector<std::string> known = COMMON;
  for (const char *k : {"temperature", "top-k", "top-p", "max-new-tokens", "seed"}) known.push_back(k);
  const Args a = parse_args(argc, argv, 2, known, {}, ALIAS);
  if (a.has("help")) {
    fprintf(stderr, "Usage: llm chat -m FOLDER [options]\n");
    common_help();
    fprintf(stderr, "  --temperature T --top-k K --top-p P --max-new-tokens N --seed S\n");
    return 0;
  }
  Model model;
  load_model(a, &model);
  printf("Please input your question (token ids).\n");
  printf("    Type ':new' to start a new session (clean history).\n");
  printf("    Type ':sys <ids>' to set the system prompt and start a new session .\n");
  std::vector<long long> history, system;
  long long turn = 0;
  const long long seed = atoll(a.get("seed", "0").c_str());
  std::string line;
  for (;;) {
    printf("> ");
    fflush(stdout);
    if (!std::getline(std::cin, line)) {
      printf("\n");
      break;
    }
    while (!line.empty() && (line.back() == '\n' || line.back() == '\r' || line.back() == ' ')) line.pop_back();
    size_t b = 0;
    while (b < line.size() && line[b] == ' ') ++b;
    const std::string q = line.substr(b);
    std::string lower = q.substr(0, 5);
    for (auto &c : lower) c = (char)tolower(c);
    if (q.size() > 5 && lower == ":sys ") {
      try {
        system = parse_ids(q.substr(5));
        history.clear();
      } catch (const Fail &f) {
        fprintf(stderr, "%s\n", f.message.c_str());
      }
      continue;
    }
    if (lower == ":new" && q.size() == 4) {
      printf("===== new session =====\n");
      history.clear();
      continue;
    }
    if (q.empty()) continue;
    std::vector<long long> ids;
    try {
      ids = parse_ids(q);
    } catch (const Fail &) {
      fprintf(stderr, "a line is a list of token ids, ':new' or ':sys <ids>'\n");
      continue;
    }
    if (history.empty() && !system.empty()) history = system;
    history.insert(history.end(), ids.begin(), ids.end());
    const double t0 = now();
    JsonHandle kwargs("{\"prompt_ids\": " + ids_json(history) + ", \"temperature\": " + a.get("temperature", "1.0") +
                      ", \"top_k\": " + a.get("top-k", "50") + ", \"top_p\": " + a.get("top-p", "0.8") + ", \"max_new_tokens\": " +
                      a.get("max-new-tokens", "256") + ", \"seed\": " + std::to_string(seed + turn) + "}");
    llm_completion_t comp = nullptr;
    check(llm_completion_init(&comp));
    std::vector<long long> answer;
    try {
      check(llm_model_complete(&model.m, &kwargs.j, &comp));
      JsonHandle chunk;
      for (;;) {
        const int32_t st = llm_completion_get_next_chunk(&comp, &chunk.j);
        if (st == LLM_ERROR_EOF) break;
        check(st);
        // {"token": id, "text": "<id>"}
        const std::string text = chunk.dump();
        const size_t p = text.find("\"token\":");
        const long long tok = atoll(text.c_str() + p + 8);
        printf("%lld ", tok);
        fflush(stdout);
        answer.push_back(tok);
      }
    } catch (const Fail &f) {
      llm_completion_destroy(&comp);
      fprintf(stderr, "\nllm: %s\n", f.message.c_str());
      continue;
    }
    llm_completion_destroy(&comp);
    printf("\n");
    history.insert(history.end(), answer.begin(), answer.end());
    ++turn;
    const double dur = now() - t0;
    const size_t n = answer.empty() ? 1 : answer.size();
    printf("(%zu tokens, time=%.2fs, %.2fms per token)\n", answer.size(), dur, dur * 1000 / (double)n);
  }
  return 0;
}

int generate_main(int argc, char **argv) {
  std::vector<std::string> known = COMMON;
  for (const char *k : {"prompt-ids", "max-new-tokens", "temperature", "top-k", "top-p", "seed", "stop-ids", "max-batch"}) known.push_back(k);
  const Args a = parse_args(argc, argv, 2, known, {"no-stop"}, ALIAS);
  if (a.has("help")) {
    fprintf(stderr, "Usage: llm generate -m FOLDER --prompt-ids 1,2,3 [--prompt-ids ...] [options]\n");
    common_help();
    fprintf(stderr,
            "  --prompt-ids IDS         a prompt as token ids; may be repeated\n"
            "  --max-new-tokens N       (default 64)\n"
            "  --temperature T          0 is greedy (default 1.0); --top-k K (50) --top-p P (0.8) --seed S (0)\n"
            "  --no-stop                ignore the model's stop tokens; --stop-ids IDS: stop tokens instead of the model's own\n");
    return 0;
  }
  if (!a.has("prompt-ids")) throw Fail{"at least one --prompt-ids is required"};
  std::string prompts = "[";
  for (size_t i = 0; i < a.values.at("prompt-ids").size(); ++i)
    prompts += (i ? "," : "") + ids_json(parse_ids(a.values.at("prompt-ids")[i]));
  prompts += "]";
  Model model;
  load_model(a, &model);
  std::string kw = "{\"prompts\": " + prompts + ", \"max_new_tokens\": " + a.get("max-new-tokens", "64") + ", \"temperature\": " +
                   a.get("temperature", "1.0") + ", \"top_k\": " + a.get("top-k", "50") + ", \"top_p\": " + a.get("top-p", "0.8") +
                   ", \"seed\": " + a.get("seed", "0") + ", \"max_batch\": " + a.get("max-batch", "64");
  if (a.has("no-stop")) kw += ", \"stop_token_ids\": []";
  else if (a.has("stop-ids")) kw += ", \"stop_token_ids\": " + ids_json(parse_ids(a.get("stop-ids", "")));
  kw += "}";
  JsonHandle kwargs(kw), result;
  const double t0 = now();
  check(llm_model_generate(&model.m, &kwargs.j, nullptr, nullptr, &result.j));
  const double dur = now() - t0;
  // {"tokens":[[...],[...]]}: one line of ids per prompt
  const std::string text = result.dump();
  size_t n = 0, p = text.find('[');
  std::string lines;
  int depth = 0;
  std::string cur;
  for (size_t i = p; i < text.size(); ++i) {
    const char c = text[i];
    if (c == '[') {
      ++depth;
      cur.clear();
    } else if (c == ']') {
      if (depth == 2) {
        lines += cur + "\n";
        for (char d : cur) n += d == ',';
        n += !cur.empty();
      }
      --depth;
    } else if (depth == 2 && c != ' ') {
      cur.push_back(c);
    }
  }
  fprintf(stderr, "(%zu tokens, time=%.2fs, %.2fms per token)\n", n, dur, dur * 1000 / (double)(n ? n : 1));
  fputs(lines.c_str(), stdout);
  return 0;
}

}  // namespace

int main(int argc, char **argv) {
  if (argc < 2) {
    usage();
    return 1;
  }
  llm_init();
  const std::string command = argv[1];
  try {
    if (command == "chat") return chat_main(argc, argv);
    if (command == "generate") return generate_main(argc, argv);
  } catch (const Fail &f) {
    fprintf(stderr, "llm: %s\n", f.message.c_str());
    return 1;
  }
  fprintf(stderr, "Invalid command \"%s\"\n\n", command.c_str());
  usage();
  return 1;
}
