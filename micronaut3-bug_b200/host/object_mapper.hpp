/*
 * object_mapper.hpp — host-side C++ mirror of the serde surface the reference uses, on top of the C ABI.
 *
 * The reference (Java) reaches this path through io.micronaut.serde.ObjectMapper:
 *   objectMapper.readValue(stream, ConfigData.class)   src/main/java/com/micronaut/bug/config/MyEntityConfig.java:34
 *   ObjectMapper.getDefault()                          src/main/java/com/micronaut/bug/service/MyEntityService.java:45
 *   response body encoding of a @Serdeable value       src/main/java/com/micronaut/bug/controller/MyEntityController.java:48-51
 * and the models the OpenAPI generator would emit for petstore.json:823-972. A JVM is not available
 * where this is built, so the same surface is written in C++: same method names, same argument meaning,
 * and a SerdeException (the reference's calls throw IOException subclasses, MyEntityService.java:3)
 * carrying the failure kind and byte offset. Every call goes to the CUDA kernels through libpetjson.so;
 * nothing is parsed or formatted on the host.
 */
#ifndef PETJSON_OBJECT_MAPPER_HPP
#define PETJSON_OBJECT_MAPPER_HPP

#include <cstdint>
#include <cstring>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "petjson.h"

namespace petjson {

/* ---- the generated models (petstore.json:823-972) ------------------------------------------------- */
struct Category { std::optional<int64_t> id; std::optional<std::string> name; };
struct Tag { std::optional<int64_t> id; std::optional<std::string> name; };
enum class PetStatus : uint8_t { AVAILABLE = 0, PENDING = 1, SOLD = 2 };
struct Pet {
  std::optional<int64_t> id;
  std::optional<Category> category;
  std::string name;                    /* required, petstore.json:873-876 */
  std::vector<std::string> photoUrls;  /* required */
  std::optional<std::vector<Tag>> tags;
  std::optional<PetStatus> status;
};
enum class OrderStatus : uint8_t { PLACED = 0, APPROVED = 1, DELIVERED = 2 };
struct OffsetDateTime { int64_t epochSecond; int32_t nano; int32_t offsetSeconds; };
struct Order {
  std::optional<int64_t> id, petId;
  std::optional<int32_t> quantity;
  std::optional<OffsetDateTime> shipDate;
  std::optional<OrderStatus> status;
  std::optional<bool> complete;
};
struct User {
  std::optional<int64_t> id;
  std::optional<std::string> username, firstName, lastName, email, password, phone;
  std::optional<int32_t> userStatus;
};

/* What a failed readValue throws: the validation kind (PJ_E_*), the record and the byte offset in it. */
class SerdeException : public std::runtime_error {
 public:
  SerdeException(int kind, uint64_t record, uint64_t offset)
      : std::runtime_error(std::string("JSON record ") + std::to_string(record) + ": " + pj_error_kind_str(kind) + " at byte " + std::to_string(offset)),
        kind(kind), record(record), offset(offset) {}
  int kind;
  uint64_t record, offset;
};
/* A failed call of the library itself (no device, out of memory, ...). */
class MapperError : public std::runtime_error {
 public:
  MapperError(pj_status st, const std::string& what) : std::runtime_error(what + ": " + pj_status_str(st)), status(st) {}
  pj_status status;
};

template <class T> struct ModelOf;
template <> struct ModelOf<Pet> { static constexpr uint32_t schema = PJ_SCHEMA_PET; };
template <> struct ModelOf<Order> { static constexpr uint32_t schema = PJ_SCHEMA_ORDER; };
template <> struct ModelOf<User> { static constexpr uint32_t schema = PJ_SCHEMA_USER; };

/* Host-memory column set with owned storage. */
class Columns {
 public:
  pj_columns raw{};
  explicit Columns(uint32_t schema) { raw.schema = schema; raw.mem_kind = PJ_MEM_HOST; }
  void reserve(uint64_t max_records, uint64_t max_input_bytes) {
    pj_columns probe{};
    if (pj_status st = pj_columns_sizes(raw.schema, max_records, max_input_bytes, 0, &probe)) throw MapperError(st, "pj_columns_sizes");
    for (int c = 0; c < PJ_MAX_COLS; ++c) if (probe.col[c].bytes) set(c, probe.col[c].bytes);
  }
  void set(int col, uint64_t bytes) {
    store_[col].assign(bytes + 16, 0);
    raw.col[col].ptr = store_[col].data(); raw.col[col].bytes = bytes; raw.col[col].count = 0;
  }
  template <class U> const U* at(int col) const { return reinterpret_cast<const U*>(raw.col[col].ptr); }
  template <class U> U* at(int col) { return reinterpret_cast<U*>(raw.col[col].ptr); }
  template <class U> void push(int col, U v) {
    auto& s = store_[col];
    size_t n = (size_t)raw.col[col].count * sizeof(U);
    if (s.size() < n + sizeof(U) + 16) s.resize((n + sizeof(U)) * 2 + 64);
    std::memcpy(s.data() + n, &v, sizeof(U));
    raw.col[col].ptr = s.data(); raw.col[col].bytes = s.size(); raw.col[col].count++;
  }
  void push_str(int off_col, const std::string* s) { /* appends to (off_col, off_col + 1) */
    if (raw.col[off_col].count == 0) push<uint32_t>(off_col, 0);
    if (s) for (char ch : *s) push<uint8_t>(off_col + 1, (uint8_t)ch);
    push<uint32_t>(off_col, (uint32_t)raw.col[off_col + 1].count);
  }
  std::string str(int off_col, uint64_t row) const {
    const uint32_t* off = at<uint32_t>(off_col);
    return std::string(reinterpret_cast<const char*>(at<uint8_t>(off_col + 1)) + off[row], off[row + 1] - off[row]);
  }

 private:
  std::vector<uint8_t> store_[PJ_MAX_COLS];
};

class ObjectMapper {
 public:
  /* ObjectMapper.getDefault(): one process-wide mapper on the current CUDA device, NON_EMPTY inclusion. */
  static ObjectMapper& getDefault() { static ObjectMapper m; return m; }

  explicit ObjectMapper(int device = -1, int inclusion = PJ_INCLUDE_NON_EMPTY) {
    pj_options opt{};
    opt.device = device; opt.inclusion = inclusion;
    if (pj_status st = pj_create(&opt, &ctx_)) throw MapperError(st, std::string("pj_create: ") + pj_last_error(nullptr));
  }
  ~ObjectMapper() { pj_destroy(ctx_); }
  ObjectMapper(const ObjectMapper&) = delete;
  ObjectMapper& operator=(const ObjectMapper&) = delete;

  /* readValue(byte[], Class<T>): one JSON document holding one record. Throws SerdeException. */
  template <class T> T readValue(const std::string& json) {
    std::string line = json;
    for (char& ch : line) if (ch == '\n') ch = ' '; /* one record per call: a line break is just whitespace */
    auto all = readValues<T>(reinterpret_cast<const uint8_t*>(line.data()), line.size());
    if (all.empty()) throw SerdeException(PJ_E_EOF, 0, line.size()); /* "No content to map due to end-of-input" */
    return std::move(all.front());
  }
  /* readValue(byte[], Argument.listOf(T)): a batch, one record per line. Throws on the first failed record. */
  template <class T> std::vector<T> readValues(const uint8_t* ndjson, uint64_t len) {
    Columns cols(ModelOf<T>::schema);
    parse(ndjson, len, cols);
    const uint8_t* kind = cols.at<uint8_t>(PJ_COL_ERR_KIND);
    const uint32_t* off = cols.at<uint32_t>(PJ_COL_ERR_OFF);
    std::vector<T> out;
    out.reserve(cols.raw.n_records);
    for (uint64_t i = 0; i < cols.raw.n_records; ++i) {
      if (kind[i]) throw SerdeException(kind[i], i, off[i]);
      out.push_back(materialise<T>(cols, i));
    }
    return out;
  }
  /* The columnar form itself, failures as data (err_kind / err_off), for callers that do not want objects. */
  void parse(const uint8_t* ndjson, uint64_t len, Columns& cols) {
    uint64_t lines = 2;
    for (uint64_t i = 0; i < len; ++i) lines += ndjson[i] == '\n';
    cols.reserve(lines, len);
    if (pj_status st = pj_parse(ctx_, cols.raw.schema, PJ_FRAMING_NDJSON, ndjson, len, PJ_MEM_HOST, &cols.raw))
      throw MapperError(st, std::string("pj_parse: ") + pj_last_error(ctx_));
  }
  /* writeValueAsString(T) / writeValueAsBytes(List<T>) */
  template <class T> std::string writeValueAsString(const T& value) {
    std::string s = writeValuesAsString(std::vector<T>{value});
    if (!s.empty() && s.back() == '\n') s.pop_back();
    return s;
  }
  template <class T> std::string writeValuesAsString(const std::vector<T>& values, uint32_t framing = PJ_FRAMING_NDJSON) {
    Columns cols(ModelOf<T>::schema);
    for (const T& v : values) append(cols, v);
    close(cols, (T*)nullptr);
    cols.raw.n_records = values.size();
    cols.raw.n_rows[ModelOf<T>::schema] = values.size();
    uint64_t need = 0;
    pj_status st = pj_write(ctx_, cols.raw.schema, framing, &cols.raw, nullptr, 0, PJ_MEM_HOST, &need);
    if (st != PJ_OK && st != PJ_ERR_CAPACITY) throw MapperError(st, std::string("pj_write: ") + pj_last_error(ctx_));
    std::string out(need, '\0');
    if (need) {
      st = pj_write(ctx_, cols.raw.schema, framing, &cols.raw, reinterpret_cast<uint8_t*>(&out[0]), need, PJ_MEM_HOST, &need);
      if (st) throw MapperError(st, std::string("pj_write: ") + pj_last_error(ctx_));
    }
    return out;
  }

 private:
  pj_ctx* ctx_ = nullptr;

  template <class T> static T materialise(const Columns& c, uint64_t r);
  static void append(Columns& c, const Pet& p);
  static void append(Columns& c, const Order& o);
  static void append(Columns& c, const User& u);
  static void close(Columns& c, Pet*) {
    for (int col : {PJ_COL_PET_CAT_NAME_OFF, PJ_COL_PET_NAME_OFF, PJ_COL_PET_PHOTO_OFF, PJ_COL_PET_PHOTO_STR_OFF, PJ_COL_PET_TAGS_OFF, PJ_COL_PET_TAG_NAME_OFF})
      if (c.raw.col[col].count == 0) c.push<uint32_t>(col, 0);
  }
  static void close(Columns&, Order*) {}
  static void close(Columns& c, User*) {
    for (int f = 0; f < 6; ++f) if (c.raw.col[PJ_COL_USR_USERNAME_OFF + 2 * f].count == 0) c.push<uint32_t>(PJ_COL_USR_USERNAME_OFF + 2 * f, 0);
  }
};

/* ---- columns -> objects ---------------------------------------------------------------------------- */
template <> inline Pet ObjectMapper::materialise<Pet>(const Columns& c, uint64_t r) {
  Pet p;
  const uint8_t pr = c.at<uint8_t>(PJ_COL_PET_PRESENT)[r];
  if (pr & 1) p.id = c.at<int64_t>(PJ_COL_PET_ID)[r];
  if (pr & 2) {
    Category cat;
    const uint8_t cp = c.at<uint8_t>(PJ_COL_PET_CAT_PRESENT)[r];
    if (cp & 1) cat.id = c.at<int64_t>(PJ_COL_PET_CAT_ID)[r];
    if (cp & 2) cat.name = c.str(PJ_COL_PET_CAT_NAME_OFF, r);
    p.category = cat;
  }
  p.name = c.str(PJ_COL_PET_NAME_OFF, r);
  const uint32_t* po = c.at<uint32_t>(PJ_COL_PET_PHOTO_OFF);
  for (uint32_t k = po[r]; k < po[r + 1]; ++k) p.photoUrls.push_back(c.str(PJ_COL_PET_PHOTO_STR_OFF, k));
  if (pr & 16) {
    std::vector<Tag> tags;
    const uint32_t* to = c.at<uint32_t>(PJ_COL_PET_TAGS_OFF);
    for (uint32_t k = to[r]; k < to[r + 1]; ++k) {
      Tag t;
      const uint8_t tp = c.at<uint8_t>(PJ_COL_PET_TAG_PRESENT)[k];
      if (tp & 1) t.id = c.at<int64_t>(PJ_COL_PET_TAG_ID)[k];
      if (tp & 2) t.name = c.str(PJ_COL_PET_TAG_NAME_OFF, k);
      tags.push_back(t);
    }
    p.tags = tags;
  }
  if (pr & 32) p.status = (PetStatus)c.at<uint8_t>(PJ_COL_PET_STATUS)[r];
  return p;
}
template <> inline Order ObjectMapper::materialise<Order>(const Columns& c, uint64_t r) {
  Order o;
  const uint8_t pr = c.at<uint8_t>(PJ_COL_ORD_PRESENT)[r];
  if (pr & 1) o.id = c.at<int64_t>(PJ_COL_ORD_ID)[r];
  if (pr & 2) o.petId = c.at<int64_t>(PJ_COL_ORD_PET_ID)[r];
  if (pr & 4) o.quantity = c.at<int32_t>(PJ_COL_ORD_QUANTITY)[r];
  if (pr & 8) o.shipDate = OffsetDateTime{c.at<int64_t>(PJ_COL_ORD_SHIP_EPOCH)[r], c.at<int32_t>(PJ_COL_ORD_SHIP_NANOS)[r], c.at<int32_t>(PJ_COL_ORD_SHIP_OFFSET)[r]};
  if (pr & 16) o.status = (OrderStatus)c.at<uint8_t>(PJ_COL_ORD_STATUS)[r];
  if (pr & 32) o.complete = c.at<uint8_t>(PJ_COL_ORD_COMPLETE)[r] != 0;
  return o;
}
template <> inline User ObjectMapper::materialise<User>(const Columns& c, uint64_t r) {
  User u;
  const uint8_t pr = c.at<uint8_t>(PJ_COL_USR_PRESENT)[r];
  if (pr & 1) u.id = c.at<int64_t>(PJ_COL_USR_ID)[r];
  std::optional<std::string>* s[6] = {&u.username, &u.firstName, &u.lastName, &u.email, &u.password, &u.phone};
  for (int f = 0; f < 6; ++f) if (pr & (2 << f)) *s[f] = c.str(PJ_COL_USR_USERNAME_OFF + 2 * f, r);
  if (pr & 128) u.userStatus = c.at<int32_t>(PJ_COL_USR_STATUS)[r];
  return u;
}

/* ---- objects -> columns ---------------------------------------------------------------------------- */
inline void ObjectMapper::append(Columns& c, const Pet& p) {
  uint8_t pr = 4 | 8; /* the required properties are always present */
  if (p.id) pr |= 1;
  if (p.category) pr |= 2;
  if (p.tags) pr |= 16;
  if (p.status) pr |= 32;
  c.push<uint8_t>(PJ_COL_PET_PRESENT, pr);
  c.push<int64_t>(PJ_COL_PET_ID, p.id.value_or(0));
  uint8_t cp = 0;
  if (p.category) cp = (p.category->id ? 1 : 0) | (p.category->name ? 2 : 0);
  c.push<uint8_t>(PJ_COL_PET_CAT_PRESENT, cp);
  c.push<int64_t>(PJ_COL_PET_CAT_ID, (cp & 1) ? *p.category->id : 0);
  c.push_str(PJ_COL_PET_CAT_NAME_OFF, (cp & 2) ? &*p.category->name : nullptr);
  c.push_str(PJ_COL_PET_NAME_OFF, &p.name);
  if (c.raw.col[PJ_COL_PET_PHOTO_OFF].count == 0) c.push<uint32_t>(PJ_COL_PET_PHOTO_OFF, 0);
  for (const auto& u : p.photoUrls) c.push_str(PJ_COL_PET_PHOTO_STR_OFF, &u);
  const uint64_t nphoto = c.raw.col[PJ_COL_PET_PHOTO_STR_OFF].count ? c.raw.col[PJ_COL_PET_PHOTO_STR_OFF].count - 1 : 0;
  c.push<uint32_t>(PJ_COL_PET_PHOTO_OFF, (uint32_t)nphoto);
  if (c.raw.col[PJ_COL_PET_TAGS_OFF].count == 0) c.push<uint32_t>(PJ_COL_PET_TAGS_OFF, 0);
  if (p.tags) for (const auto& t : *p.tags) {
    c.push<uint8_t>(PJ_COL_PET_TAG_PRESENT, (uint8_t)((t.id ? 1 : 0) | (t.name ? 2 : 0)));
    c.push<int64_t>(PJ_COL_PET_TAG_ID, t.id.value_or(0));
    c.push_str(PJ_COL_PET_TAG_NAME_OFF, t.name ? &*t.name : nullptr);
  }
  c.push<uint32_t>(PJ_COL_PET_TAGS_OFF, (uint32_t)c.raw.col[PJ_COL_PET_TAG_PRESENT].count);
  c.push<uint8_t>(PJ_COL_PET_STATUS, p.status ? (uint8_t)*p.status : 255);
}
inline void ObjectMapper::append(Columns& c, const Order& o) {
  uint8_t pr = (o.id ? 1 : 0) | (o.petId ? 2 : 0) | (o.quantity ? 4 : 0) | (o.shipDate ? 8 : 0) | (o.status ? 16 : 0) | (o.complete ? 32 : 0);
  c.push<uint8_t>(PJ_COL_ORD_PRESENT, pr);
  c.push<int64_t>(PJ_COL_ORD_ID, o.id.value_or(0));
  c.push<int64_t>(PJ_COL_ORD_PET_ID, o.petId.value_or(0));
  c.push<int32_t>(PJ_COL_ORD_QUANTITY, o.quantity.value_or(0));
  c.push<int64_t>(PJ_COL_ORD_SHIP_EPOCH, o.shipDate ? o.shipDate->epochSecond : 0);
  c.push<int32_t>(PJ_COL_ORD_SHIP_NANOS, o.shipDate ? o.shipDate->nano : 0);
  c.push<int32_t>(PJ_COL_ORD_SHIP_OFFSET, o.shipDate ? o.shipDate->offsetSeconds : 0);
  c.push<uint8_t>(PJ_COL_ORD_STATUS, o.status ? (uint8_t)*o.status : 255);
  c.push<uint8_t>(PJ_COL_ORD_COMPLETE, o.complete.value_or(false) ? 1 : 0);
}
inline void ObjectMapper::append(Columns& c, const User& u) {
  const std::optional<std::string>* s[6] = {&u.username, &u.firstName, &u.lastName, &u.email, &u.password, &u.phone};
  uint8_t pr = (u.id ? 1 : 0) | (u.userStatus ? 128 : 0);
  for (int f = 0; f < 6; ++f) if (*s[f]) pr |= (uint8_t)(2 << f);
  c.push<uint8_t>(PJ_COL_USR_PRESENT, pr);
  c.push<int64_t>(PJ_COL_USR_ID, u.id.value_or(0));
  for (int f = 0; f < 6; ++f) c.push_str(PJ_COL_USR_USERNAME_OFF + 2 * f, *s[f] ? &**s[f] : nullptr);
  c.push<int32_t>(PJ_COL_USR_STATUS, u.userStatus.value_or(0));
}

}  // namespace petjson
#endif
