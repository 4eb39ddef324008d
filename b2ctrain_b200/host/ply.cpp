// Splat PLY files (the 3DGS layout the reference reads and writes, src/ply.cpp:80-226): x y z, scale_0..2 (log),
// opacity (logit), rot_0..3 (w x y z), f_dc_0..2, f_rest_* channel-major, optional per-splat evidence (ev_*) and label
// (seg_*) columns. Reader: ascii or binary little-endian, any scalar property types, vertex element only; a cloud without
// f_dc takes its base colour from red/green/blue. Writer: binary little-endian float32, quaternions normalised.
//
// Organisation: the header is compiled into a list of (source offset, type, destination) moves, so a row is decoded by
// one pass over that list straight into the cloud's arrays.
#include <cmath>
#include <cstring>
#include <fstream>
#include <sstream>
#include "b2c_api.h"

namespace b2c {

const char* const EVIDENCE_FIELDS[7] = {"ev_w_in", "ev_w_all", "ev_err", "ev_views", "ev_dir_0", "ev_dir_1", "ev_dir_2"};
const char* const LABEL_FIELDS[2] = {"seg_label", "seg_conf"};

namespace {

[[noreturn]] void ply_fail(const std::string& msg) { throw std::runtime_error("ply: " + msg); }

enum Scalar { S_F32, S_F64, S_U8, S_I8, S_U16, S_I16, S_U32, S_I32 };

struct Column { std::string name; Scalar type; size_t offset; };

Scalar scalar_of(const std::string& t) {
  static const struct { const char* a; const char* b; Scalar s; } names[] = {
      {"float", "float32", S_F32}, {"double", "float64", S_F64}, {"uchar", "uint8", S_U8}, {"char", "int8", S_I8},
      {"ushort", "uint16", S_U16}, {"short", "int16", S_I16}, {"uint", "uint32", S_U32}, {"int", "int32", S_I32}};
  for (const auto& n : names) if (t == n.a || t == n.b) return n.s;
  ply_fail("unsupported property type '" + t + "'");
}
size_t width_of(Scalar s) { return s == S_F64 ? 8 : (s == S_F32 || s == S_U32 || s == S_I32) ? 4 : (s == S_U16 || s == S_I16) ? 2 : 1; }

double decode(const unsigned char* p, Scalar s) {
  switch (s) {
    case S_F32: { float v; std::memcpy(&v, p, 4); return v; }
    case S_F64: { double v; std::memcpy(&v, p, 8); return v; }
    case S_U8: return (double)*p;
    case S_I8: return (double)(signed char)*p;
    case S_U16: { uint16_t v; std::memcpy(&v, p, 2); return v; }
    case S_I16: { int16_t v; std::memcpy(&v, p, 2); return v; }
    case S_U32: { uint32_t v; std::memcpy(&v, p, 4); return v; }
    default: { int32_t v; std::memcpy(&v, p, 4); return v; }
  }
}

struct Header {
  bool ascii = false;
  size_t n = 0, row_bytes = 0;
  std::vector<Column> cols;
  std::vector<std::string> comments;
  const Column* find(const std::string& name) const { for (const Column& c : cols) if (c.name == name) return &c; return nullptr; }
};

Header read_header(std::istream& f, const std::string& path) {
  Header h;
  std::string line;
  if (!std::getline(f, line) || line.compare(0, 3, "ply") != 0) ply_fail("'" + path + "' is not a ply file");
  bool in_vertex = false, ended = false;
  while (std::getline(f, line)) {
    if (!line.empty() && line.back() == '\r') line.pop_back();
    std::istringstream ss(line);
    std::string key; ss >> key;
    if (key == "end_header") { ended = true; break; }
    if (key == "comment") { h.comments.push_back(line.size() > 8 ? line.substr(8) : std::string()); continue; }
    if (key == "format") {
      std::string fmt; ss >> fmt;
      if (fmt == "binary_big_endian") ply_fail("big-endian files are not supported");
      h.ascii = fmt == "ascii";
    } else if (key == "element") {
      std::string name; size_t count = 0; ss >> name >> count;
      in_vertex = name == "vertex";
      if (in_vertex) h.n = count; else if (count > 0) ply_fail("unsupported non-vertex element '" + name + "'");
    } else if (key == "property" && in_vertex) {
      std::string type, name; ss >> type;
      if (type == "list") ply_fail("list properties are not supported on vertices");
      ss >> name;
      const Scalar s = scalar_of(type);
      h.cols.push_back({name, s, h.row_bytes});
      h.row_bytes += width_of(s);
    }
  }
  if (!ended) ply_fail("'" + path + "' has no end_header");
  return h;
}

// One decoded value of a row goes to dst[row * stride + at], after `v * scale + bias`.
struct Move { size_t col; std::vector<float>* dst; size_t stride, at; double scale, bias; };

}  // namespace

bool ply_is_vertex_only(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  try { const Header h = read_header(f, path); return h.n > 0; } catch (const std::exception&) { return false; }
}

std::vector<std::string> read_ply_comments(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return {};
  try { return read_header(f, path).comments; } catch (const std::exception&) { return {}; }
}

SplatCloud read_ply(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) ply_fail("failed to open '" + path + "'");
  const Header h = read_header(f, path);
  for (const char* need : {"x", "y", "z"}) if (!h.find(need)) ply_fail("missing x/y/z");
  int n_rest = 0;
  while (h.find("f_rest_" + std::to_string(n_rest))) n_rest++;
  const int K = 1 + n_rest / 3, degree = (int)std::lround(std::sqrt((double)K)) - 1;
  if ((degree + 1) * (degree + 1) != K || n_rest % 3 != 0) ply_fail(std::to_string(n_rest) + " f_rest properties is not a valid SH layout");

  SplatCloud c;
  c.has_evidence = h.find("ev_w_in") != nullptr;
  c.has_labels = h.find("seg_label") != nullptr;
  c.resize(h.n, degree);
  for (size_t i = 0; i < c.n; i++) c.quat[i * 4] = 1.f;   // identity where the file has no rotation
  c.has_scales = h.find("scale_0") != nullptr;
  if (c.has_evidence) c.evidence.assign(c.n * 7, 0.f);
  if (c.has_labels) { c.labels.assign(c.n * 2, 0.f); for (size_t i = 0; i < c.n; i++) c.labels[i * 2 + 1] = 1.f; }

  std::vector<Move> moves;
  auto map = [&](const std::string& name, std::vector<float>& dst, size_t stride, size_t at, double scale = 1.0, double bias = 0.0) {
    for (size_t k = 0; k < h.cols.size(); k++) if (h.cols[k].name == name) { moves.push_back({k, &dst, stride, at, scale, bias}); return true; }
    return false;
  };
  const char* xyz[3] = {"x", "y", "z"};
  for (int k = 0; k < 3; k++) { map(xyz[k], c.pos, 3, k); map("scale_" + std::to_string(k), c.log_scale, 3, k); }
  for (int k = 0; k < 4; k++) map("rot_" + std::to_string(k), c.quat, 4, k);
  map("opacity", c.opacity, 1, 0);
  const size_t sh_stride = (size_t)K * 3;
  if (h.find("f_dc_0")) {
    for (int ch = 0; ch < 3; ch++) map("f_dc_" + std::to_string(ch), c.sh, sh_stride, ch);
  } else {   // base colour from 8/16-bit or float rgb: sh0 = (colour - 0.5) / C0
    const char* longn[3] = {"red", "green", "blue"}; const char* shortn[3] = {"r", "g", "b"};
    for (int ch = 0; ch < 3; ch++) {
      const Column* col = h.find(longn[ch]) ? h.find(longn[ch]) : h.find(shortn[ch]);
      if (!col) continue;
      const double unit = col->type == S_U8 ? 1.0 / 255.0 : col->type == S_U16 ? 1.0 / 65535.0 : 1.0;
      map(col->name, c.sh, sh_stride, ch, unit / SH_C0, -0.5 / SH_C0);
    }
  }
  for (int ch = 0; ch < 3; ch++)     // f_rest is channel-major: all red coefficients, then green, then blue
    for (int k = 1; k < K; k++) map("f_rest_" + std::to_string(ch * (K - 1) + (k - 1)), c.sh, sh_stride, (size_t)k * 3 + ch);
  if (c.has_evidence) for (int k = 0; k < 7; k++) map(EVIDENCE_FIELDS[k], c.evidence, 7, k);
  if (c.has_labels) for (int k = 0; k < 2; k++) map(LABEL_FIELDS[k], c.labels, 2, k);

  if (h.ascii) {
    std::vector<double> row(h.cols.size());
    for (size_t r = 0; r < h.n; r++) {
      for (double& v : row) if (!(f >> v)) ply_fail("truncated ascii file '" + path + "'");
      for (const Move& m : moves) (*m.dst)[r * m.stride + m.at] = (float)(row[m.col] * m.scale + m.bias);
    }
  } else {
    constexpr size_t ROWS = 4096;
    std::vector<unsigned char> buf(h.row_bytes * ROWS);
    for (size_t done = 0; done < h.n;) {
      const size_t take = std::min(ROWS, h.n - done);
      f.read((char*)buf.data(), (std::streamsize)(take * h.row_bytes));
      if ((size_t)f.gcount() != take * h.row_bytes)
        ply_fail("truncated file '" + path + "' (got " + std::to_string(done + (size_t)f.gcount() / std::max<size_t>(h.row_bytes, 1)) + " of " + std::to_string(h.n) + " vertices)");
      for (const Move& m : moves) {
        const Column& col = h.cols[m.col];
        const unsigned char* src = buf.data() + col.offset;
        float* dst = m.dst->data() + done * m.stride + m.at;
        for (size_t r = 0; r < take; r++) dst[r * m.stride] = (float)(decode(src + r * h.row_bytes, col.type) * m.scale + m.bias);
      }
      done += take;
    }
  }
  return c;
}

void write_ply(const std::string& path, const SplatCloud& c, const std::vector<std::string>& comments) {
  std::ofstream f(path, std::ios::binary);
  if (!f) ply_fail("failed to open '" + path + "' for writing");
  const int K = c.K(), rest = 3 * (K - 1);
  std::ostringstream head;
  head << "ply\nformat binary_little_endian 1.0\n";
  for (const std::string& cm : comments) head << "comment " << cm << "\n";
  head << "element vertex " << c.n << "\n";
  std::vector<std::string> names = {"x", "y", "z", "scale_0", "scale_1", "scale_2", "opacity", "rot_0", "rot_1", "rot_2", "rot_3", "f_dc_0", "f_dc_1", "f_dc_2"};
  for (int k = 0; k < rest; k++) names.push_back("f_rest_" + std::to_string(k));
  if (c.has_evidence) for (const char* e : EVIDENCE_FIELDS) names.push_back(e);
  if (c.has_labels) for (const char* e : LABEL_FIELDS) names.push_back(e);
  for (const std::string& nm : names) head << "property float " << nm << "\n";
  head << "end_header\n";
  const std::string hs = head.str();
  f.write(hs.data(), (std::streamsize)hs.size());
  const size_t width = names.size();
  constexpr size_t ROWS = 4096;
  std::vector<float> block(width * ROWS);
  for (size_t base = 0; base < c.n; base += ROWS) {
    const size_t take = std::min(ROWS, c.n - base);
    for (size_t r = 0; r < take; r++) {
      const size_t i = base + r;
      float* o = block.data() + r * width;
      for (int k = 0; k < 3; k++) { o[k] = c.pos[i * 3 + k]; o[3 + k] = c.log_scale[i * 3 + k]; }
      o[6] = c.opacity[i];
      const float* q = &c.quat[i * 4];
      const float len = std::sqrt(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]);
      if (len > 1e-32f) { for (int k = 0; k < 4; k++) o[7 + k] = q[k] / len; } else { o[7] = 1.f; o[8] = o[9] = o[10] = 0.f; }
      const float* sh = &c.sh[i * (size_t)K * 3];
      for (int ch = 0; ch < 3; ch++) o[11 + ch] = sh[ch];
      size_t at = 14;
      for (int ch = 0; ch < 3; ch++) for (int k = 1; k < K; k++) o[at++] = sh[k * 3 + ch];
      if (c.has_evidence) for (int k = 0; k < 7; k++) o[at++] = c.evidence[i * 7 + k];
      if (c.has_labels) { o[at++] = c.labels[i * 2]; o[at++] = c.labels[i * 2 + 1]; }
    }
    f.write((const char*)block.data(), (std::streamsize)(take * width * sizeof(float)));
  }
  if (!f) ply_fail("failed writing '" + path + "'");
}

}  // namespace b2c
