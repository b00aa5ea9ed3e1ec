// Episode dataset reader: a directory of gzip-compressed Habitat PointNav episode
// files, one scene per file.
//
// Follows Dataset / parseFile in simulator/simulator.cpp:158-359: every
// `*.json.gz` under the dataset directory holds {"episodes": [...]}, each episode
// contributes start_position[3], start_rotation[4] (x, y, z, w as stored) and
// goals[0].position[3]; all episodes of a file must name the same scene_id
// ("Loading code assumes json file contains data for one scene", :278-282); the
// navmesh of a scene is asset_path / scene_id with its extension replaced by
// ".navmesh" (:330-342).  Files are parsed on several threads as in the
// reference; unlike the reference, whose scene order depends on how its threads
// interleave, scenes are returned in file-name order.
//
// The reference parses with simdjson and inflates with zlib; simdjson is not
// part of its tree, so the small JSON reader below stands in for it.
#include "dataset_host.h"

#include <dirent.h>
#include <zlib.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <thread>

namespace bpsn {
namespace {

// ---------------------------------------------------------------- JSON (RFC 8259 subset: all of it
// except that numbers are read with strtod and \u escapes above the BMP are kept as two code units)
struct JsonValue {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<JsonValue> items;                          // Array
  std::vector<std::pair<std::string, JsonValue>> members;  // Object, in file order

  const JsonValue* get(const char* key) const {
    for (const auto& m : members)
      if (m.first == key)
        return &m.second;
    return nullptr;
  }
};

class JsonParser {
 public:
  JsonParser(const char* p, size_t n) : p_(p), end_(p + n) {}

  bool parse(JsonValue* out, std::string* err) {
    if (!value(out, 0)) {
      *err = err_.empty() ? "malformed JSON" : err_;
      return false;
    }
    ws();
    if (p_ != end_) {
      *err = "trailing characters after the JSON document";
      return false;
    }
    return true;
  }

 private:
  void ws() {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\r' || *p_ == '\t'))
      ++p_;
  }
  bool fail(const char* m) {
    if (err_.empty())
      err_ = m;
    return false;
  }
  bool literal(const char* s) {
    const size_t n = strlen(s);
    if (static_cast<size_t>(end_ - p_) < n || memcmp(p_, s, n) != 0)
      return fail("bad literal");
    p_ += n;
    return true;
  }
  static void utf8(std::string* s, unsigned cp) {
    if (cp < 0x80) {
      s->push_back(static_cast<char>(cp));
    } else if (cp < 0x800) {
      s->push_back(static_cast<char>(0xC0 | (cp >> 6)));
      s->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
      s->push_back(static_cast<char>(0xE0 | (cp >> 12)));
      s->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      s->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
  }
  bool string(std::string* out) {
    if (p_ >= end_ || *p_ != '"')
      return fail("expected a string");
    ++p_;
    out->clear();
    while (p_ < end_ && *p_ != '"') {
      char c = *p_++;
      if (c != '\\') {
        out->push_back(c);
        continue;
      }
      if (p_ >= end_)
        return fail("unterminated escape");
      c = *p_++;
      switch (c) {
        case '"': out->push_back('"'); break;
        case '\\': out->push_back('\\'); break;
        case '/': out->push_back('/'); break;
        case 'b': out->push_back('\b'); break;
        case 'f': out->push_back('\f'); break;
        case 'n': out->push_back('\n'); break;
        case 'r': out->push_back('\r'); break;
        case 't': out->push_back('\t'); break;
        case 'u': {
          if (end_ - p_ < 4)
            return fail("short \\u escape");
          unsigned cp = 0;
          for (int i = 0; i < 4; ++i) {
            const char h = *p_++;
            cp <<= 4;
            if (h >= '0' && h <= '9') cp |= static_cast<unsigned>(h - '0');
            else if (h >= 'a' && h <= 'f') cp |= static_cast<unsigned>(h - 'a' + 10);
            else if (h >= 'A' && h <= 'F') cp |= static_cast<unsigned>(h - 'A' + 10);
            else return fail("bad \\u escape");
          }
          utf8(out, cp);
          break;
        }
        default:
          return fail("bad escape");
      }
    }
    if (p_ >= end_)
      return fail("unterminated string");
    ++p_;
    return true;
  }
  bool value(JsonValue* v, int depth) {
    if (depth > 64)
      return fail("nesting too deep");
    ws();
    if (p_ >= end_)
      return fail("unexpected end of input");
    const char c = *p_;
    if (c == '{') {
      ++p_;
      v->kind = JsonValue::Object;
      ws();
      if (p_ < end_ && *p_ == '}') {
        ++p_;
        return true;
      }
      while (true) {
        ws();
        std::string key;
        if (!string(&key))
          return false;
        ws();
        if (p_ >= end_ || *p_ != ':')
          return fail("expected ':'");
        ++p_;
        v->members.emplace_back(std::move(key), JsonValue());
        if (!value(&v->members.back().second, depth + 1))
          return false;
        ws();
        if (p_ < end_ && *p_ == ',') {
          ++p_;
          continue;
        }
        if (p_ < end_ && *p_ == '}') {
          ++p_;
          return true;
        }
        return fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      ++p_;
      v->kind = JsonValue::Array;
      ws();
      if (p_ < end_ && *p_ == ']') {
        ++p_;
        return true;
      }
      while (true) {
        v->items.emplace_back();
        if (!value(&v->items.back(), depth + 1))
          return false;
        ws();
        if (p_ < end_ && *p_ == ',') {
          ++p_;
          continue;
        }
        if (p_ < end_ && *p_ == ']') {
          ++p_;
          return true;
        }
        return fail("expected ',' or ']'");
      }
    }
    if (c == '"') {
      v->kind = JsonValue::String;
      return string(&v->str);
    }
    if (c == 't') {
      v->kind = JsonValue::Bool;
      v->b = true;
      return literal("true");
    }
    if (c == 'f') {
      v->kind = JsonValue::Bool;
      v->b = false;
      return literal("false");
    }
    if (c == 'n') {
      v->kind = JsonValue::Null;
      return literal("null");
    }
    // number (also accepts what Python's json module writes for non-finite values)
    if (c == 'N' && end_ - p_ >= 3 && memcmp(p_, "NaN", 3) == 0) {
      p_ += 3;
      v->kind = JsonValue::Number;
      v->num = std::nan("");
      return true;
    }
    {
      const bool neg = c == '-';
      const char* q = p_ + (neg ? 1 : 0);
      if (end_ - q >= 8 && memcmp(q, "Infinity", 8) == 0) {
        p_ = q + 8;
        v->kind = JsonValue::Number;
        v->num = neg ? -HUGE_VAL : HUGE_VAL;
        return true;
      }
    }
    if (c == '-' || (c >= '0' && c <= '9')) {
      // copy the token: the buffer is not guaranteed to be followed by a non-number byte
      const char* q = p_;
      while (q < end_ && (strchr("+-.eE", *q) || (*q >= '0' && *q <= '9')))
        ++q;
      char tok[64];
      const size_t n = static_cast<size_t>(q - p_);
      if (n == 0 || n >= sizeof(tok))
        return fail("bad number");
      memcpy(tok, p_, n);
      tok[n] = 0;
      char* stop = nullptr;
      v->num = strtod(tok, &stop);
      if (stop != tok + n)
        return fail("bad number");
      v->kind = JsonValue::Number;
      p_ = q;
      return true;
    }
    return fail("unexpected character");
  }

  const char* p_;
  const char* end_;
  std::string err_;
};

bool inflateFile(const std::string& path, std::string* out, std::string* err) {
  gzFile f = gzopen(path.c_str(), "rb");
  if (!f) {
    *err = "Failed to open " + path;  // simulator.cpp:163-166
    return false;
  }
  out->clear();
  char buf[1 << 16];
  while (true) {
    const int n = gzread(f, buf, sizeof(buf));
    if (n < 0) {
      int code = 0;
      *err = path + ": " + gzerror(f, &code);
      gzclose(f);
      return false;
    }
    if (n == 0)
      break;
    out->append(buf, static_cast<size_t>(n));
  }
  gzclose(f);
  return true;
}

bool numbers(const JsonValue* v, int n, float* out) {
  if (!v || v->kind != JsonValue::Array || static_cast<int>(v->items.size()) < n)
    return false;
  for (int i = 0; i < n; ++i) {
    if (v->items[i].kind != JsonValue::Number)
      return false;
    out[i] = static_cast<float>(v->items[i].num);
  }
  return true;
}

bool parseEpisodeFile(const std::string& path, const std::string& assetPath, DatasetScene* scene,
                      bool* empty, std::string* err) {
  std::string text;
  if (!inflateFile(path, &text, err))
    return false;
  JsonValue doc;
  std::string perr;
  if (!JsonParser(text.data(), text.size()).parse(&doc, &perr)) {
    *err = path + ": " + perr;
    return false;
  }
  const JsonValue* eps = doc.kind == JsonValue::Object ? doc.get("episodes") : nullptr;
  if (!eps || eps->kind != JsonValue::Array) {
    *err = path + ": no \"episodes\" array";
    return false;
  }
  *empty = eps->items.empty();
  if (*empty)
    return true;
  scene->episodes.resize(eps->items.size());
  for (size_t i = 0; i < eps->items.size(); ++i) {
    const JsonValue& e = eps->items[i];
    const JsonValue* sid = e.kind == JsonValue::Object ? e.get("scene_id") : nullptr;
    if (!sid || sid->kind != JsonValue::String) {
      *err = path + ": episode " + std::to_string(i) + " has no scene_id";
      return false;
    }
    if (i == 0)
      scene->sceneId = sid->str;
    else if (sid->str != scene->sceneId) {
      *err = "Loading code assumes json file contains data for one scene";
      return false;
    }
    bpsn_episode& ep = scene->episodes[i];
    const JsonValue* goals = e.get("goals");
    const JsonValue* goal0 = goals && goals->kind == JsonValue::Array && !goals->items.empty() &&
                                     goals->items[0].kind == JsonValue::Object
                                 ? goals->items[0].get("position") : nullptr;
    if (!numbers(e.get("start_position"), 3, ep.start_position) ||
        !numbers(e.get("start_rotation"), 4, ep.start_rotation) || !numbers(goal0, 3, ep.goal)) {
      *err = path + ": episode " + std::to_string(i) +
             " lacks start_position[3], start_rotation[4] or goals[0].position[3]";
      return false;
    }
  }
  const size_t dot = scene->sceneId.rfind('.');
  if (dot == std::string::npos) {
    *err = "Invalid scene id: " + scene->sceneId;
    return false;
  }
  scene->navmeshPath = assetPath + "/" + scene->sceneId.substr(0, dot) + ".navmesh";
  return true;
}

}  // namespace

bool loadDataset(const std::string& datasetPath, const std::string& assetPath,
                 uint32_t numThreads, std::vector<DatasetScene>* out, std::string* err) {
  std::vector<std::string> files;
  DIR* d = opendir(datasetPath.c_str());
  if (!d) {
    *err = "cannot open dataset directory " + datasetPath;
    return false;
  }
  while (dirent* ent = readdir(d)) {
    const std::string name = ent->d_name;
    const char* suffix = ".json.gz";
    if (name.size() > strlen(suffix) &&
        name.compare(name.size() - strlen(suffix), strlen(suffix), suffix) == 0)
      files.push_back(name);
  }
  closedir(d);
  if (files.empty()) {
    *err = "no *.json.gz episode files under " + datasetPath;
    return false;
  }
  std::sort(files.begin(), files.end());
  std::vector<DatasetScene> scenes(files.size());
  std::vector<char> isEmpty(files.size(), 0), failed(files.size(), 0);
  std::vector<std::string> errors(files.size());
  std::atomic<size_t> next{0};
  auto work = [&]() {
    while (true) {
      const size_t i = next.fetch_add(1);
      if (i >= files.size())
        break;
      bool empty = false;
      if (!parseEpisodeFile(datasetPath + "/" + files[i], assetPath, &scenes[i], &empty,
                            &errors[i]))
        failed[i] = 1;
      isEmpty[i] = empty ? 1 : 0;
    }
  };
  uint32_t nt = numThreads ? numThreads : 1;
  if (nt > files.size())
    nt = static_cast<uint32_t>(files.size());
  std::vector<std::thread> pool;
  for (uint32_t t = 1; t < nt; ++t)
    pool.emplace_back(work);
  work();  // the calling thread takes part, as in the reference
  for (auto& th : pool)
    th.join();
  out->clear();
  for (size_t i = 0; i < files.size(); ++i) {
    if (failed[i]) {
      *err = errors[i];
      return false;
    }
    if (!isEmpty[i])
      out->push_back(std::move(scenes[i]));
  }
  return true;
}

}  // namespace bpsn
