// Profile dictionaries on disk: the cost model the scheduler plans with.  The file format is the
// reference's (src/utils.h:106-215): a JSON array of
//   {"kernel_name": int, "batch_size": int, "seq_len": int, "duration": float}            (Main)
//   {"kernel_name": int, "batch_size": int, "seq_len": int, "duration": [float, ...]}     (Sub)
// written by rank 0 and read by every rank.  The reference reads with nlohmann-json and writes by
// hand (an empty dictionary produces invalid JSON there, src/utils.h:117); both directions are
// hand-written here, an empty dictionary is "[]", and malformed input raises std::runtime_error.
#pragma once
#include <cctype>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <string>

#include "context.h"

namespace liger_host {

inline std::string profile_file_name(const char* prefix, const BertInitParam& bp, int world_size) {
  // ./Main_<ws>_<size_per_head>_<head_num>_<max_batch>_<max_seq>.json  (src/test_schedule.h:36-39)
  std::ostringstream ss;
  ss << "./" << prefix << "_" << world_size << "_" << bp.size_per_head << "_" << bp.head_num << "_"
     << bp.max_batch_size << "_" << bp.max_seq_len << ".json";
  return ss.str();
}

inline void write_text_file(const std::string& filename, const std::string& text) {
  std::ofstream f(filename);
  if (!f.is_open()) throw std::runtime_error("unable to open file " + filename);
  f << text;
}

inline void MainDictToFile(const MainDict& data, const std::string& filename) {
  std::ostringstream ss;
  ss << "[";
  bool first = true;
  for (const auto& e : data) {
    if (!first) ss << ",";
    first = false;
    ss << "{\"kernel_name\":" << e.first.kernel_name << ",\"batch_size\":" << e.first.batch_size
       << ",\"seq_len\":" << e.first.seq_len << ",\"duration\":" << e.second << "}";
  }
  ss << "]";
  write_text_file(filename, ss.str());
}

inline void SubDictToFile(const SubDict& data, const std::string& filename) {
  std::ostringstream ss;
  ss << "[";
  bool first = true;
  for (const auto& e : data) {
    if (!first) ss << ",";
    first = false;
    ss << "{\"kernel_name\":" << e.first.kernel_name << ",\"batch_size\":" << e.first.batch_size
       << ",\"seq_len\":" << e.first.seq_len << ",\"duration\": [";
    for (size_t i = 0; i < e.second.size(); ++i) ss << (i ? "," : "") << e.second[i];
    ss << "]}";
  }
  ss << "]";
  write_text_file(filename, ss.str());
}

// ---- a minimal JSON reader for exactly this schema ------------------------------------------------------
class ProfileParser {
 public:
  explicit ProfileParser(const std::string& text) : s_(text) {}
  // calls on_entry(kernel_info, scalar_duration, vector_duration, is_vector) per array element
  template <typename F>
  void parse(F on_entry) {
    ws();
    expect('[');
    ws();
    if (peek() == ']') { ++i_; return; }
    for (;;) {
      parse_object(on_entry);
      ws();
      if (peek() == ',') { ++i_; ws(); continue; }
      expect(']');
      break;
    }
  }

 private:
  const std::string& s_;
  size_t i_ = 0;
  char peek() const { return i_ < s_.size() ? s_[i_] : '\0'; }
  void ws() { while (i_ < s_.size() && isspace((unsigned char)s_[i_])) ++i_; }
  [[noreturn]] void fail(const std::string& what) const {
    throw std::runtime_error("profile JSON: " + what + " at offset " + std::to_string(i_));
  }
  void expect(char c) { if (peek() != c) fail(std::string("expected '") + c + "'"); ++i_; }
  std::string parse_string() {
    expect('"');
    std::string out;
    while (i_ < s_.size() && s_[i_] != '"') out.push_back(s_[i_++]);
    expect('"');
    return out;
  }
  double parse_number() {
    const char* b = s_.c_str() + i_;
    char* e = nullptr;
    double v = strtod(b, &e);
    if (e == b) fail("expected a number");
    i_ += (size_t)(e - b);
    return v;
  }
  template <typename F>
  void parse_object(F on_entry) {
    expect('{');
    kernel_info key{-1, -1, -1};
    bool have[4] = {false, false, false, false};
    float scalar = 0.0f;
    std::vector<float> vec;
    bool is_vec = false;
    for (;;) {
      ws();
      std::string k = parse_string();
      ws(); expect(':'); ws();
      if (k == "kernel_name") { key.kernel_name = (int)parse_number(); have[0] = true; }
      else if (k == "batch_size") { key.batch_size = (int)parse_number(); have[1] = true; }
      else if (k == "seq_len") { key.seq_len = (int)parse_number(); have[2] = true; }
      else if (k == "duration") {
        have[3] = true;
        if (peek() == '[') {
          is_vec = true;
          ++i_; ws();
          if (peek() == ']') { ++i_; }
          else for (;;) {
            vec.push_back((float)parse_number());
            ws();
            if (peek() == ',') { ++i_; ws(); continue; }
            expect(']');
            break;
          }
        } else {
          scalar = (float)parse_number();
        }
      } else fail("unknown key \"" + k + "\"");
      ws();
      if (peek() == ',') { ++i_; continue; }
      expect('}');
      break;
    }
    if (!(have[0] && have[1] && have[2] && have[3])) fail("entry is missing a key");
    on_entry(key, scalar, vec, is_vec);
  }
};

inline std::string read_text_file(const std::string& filename) {
  std::ifstream f(filename);
  if (!f.is_open()) throw std::runtime_error("unable to open file " + filename);
  std::stringstream b;
  b << f.rdbuf();
  return b.str();
}

inline MainDict MainTextToDict(const std::string& text) {
  MainDict d;
  ProfileParser p(text);
  p.parse([&](const kernel_info& k, float scalar, const std::vector<float>&, bool is_vec) {
    if (is_vec) throw std::runtime_error("profile JSON: Main file entry holds an array duration");
    d[k] = scalar;
  });
  return d;
}
inline SubDict SubTextToDict(const std::string& text) {
  SubDict d;
  ProfileParser p(text);
  p.parse([&](const kernel_info& k, float, const std::vector<float>& vec, bool is_vec) {
    if (!is_vec) throw std::runtime_error("profile JSON: Sub file entry holds a scalar duration");
    d[k] = vec;
  });
  return d;
}
inline MainDict MainFileToDict(const std::string& filename) { return MainTextToDict(read_text_file(filename)); }
inline SubDict SubFileToDict(const std::string& filename) { return SubTextToDict(read_text_file(filename)); }


// The cost model behind Scheduler::lookup_duration (see there): exact key, else linear interpolation between the
// nearest profiled lengths of the same batch size, proportional extrapolation beyond the last one, the nearest
// profiled batch size scaled by tokens otherwise; 0 when the kernel was never profiled.
inline float predict_duration(const MainDict& dict, int name, int bs, int sq, int max_bs, int max_sq) {
  auto it = dict.find({name, bs, sq});
  if (it != dict.end()) return it->second;
  int lo = 0, hi = 0;
  float dlo = 0.0f, dhi = 0.0f;
  for (int s = sq - 1; s >= 1; --s) {
    it = dict.find({name, bs, s});
    if (it != dict.end()) { lo = s; dlo = it->second; break; }
  }
  for (int s = sq + 1; s <= max_sq; ++s) {
    it = dict.find({name, bs, s});
    if (it != dict.end()) { hi = s; dhi = it->second; break; }
  }
  if (lo && hi) return dlo + (dhi - dlo) * (float)(sq - lo) / (float)(hi - lo);
  if (hi) return dhi;  // shorter than anything profiled: a floor, not a line through 0
  if (lo) return dlo * (float)sq / (float)lo;
  for (int d = 1; d <= max_bs; ++d) {
    const int cand[2] = {bs + d, bs - d};
    for (int b : cand) {
      if (b < 1 || b > max_bs) continue;
      bool any = false;
      for (int s = 1; s <= max_sq && !any; ++s) any = dict.count({name, b, s}) != 0;
      if (any) return predict_duration(dict, name, b, sq, max_bs, max_sq) * (float)bs / (float)b;
    }
  }
  return 0.0f;
}

}  // namespace liger_host
