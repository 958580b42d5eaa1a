// Self-checking use of the C++ ObjectMapper mirror (needs a CUDA device): the calls a user of the
// reference's serde surface would make, on the Petstore models.
#include <cstdio>
#include <cstdlib>

#include "object_mapper.hpp"

using namespace petjson;

#define CHECK(cond) do { if (!(cond)) { std::fprintf(stderr, "check failed at line %d: %s\n", __LINE__, #cond); return 1; } } while (0)

int main() {
  ObjectMapper& om = ObjectMapper::getDefault();

  const std::string doc =
      "{\"id\":7,\"category\":{\"id\":2,\"name\":\"dogs\"},\"name\":\"rex\",\"photoUrls\":[\"http://x/1\",\"http://x/2\"],"
      "\"tags\":[{\"id\":1,\"name\":\"good\"}],\"status\":\"pending\"}";
  Pet p = om.readValue<Pet>(doc);
  CHECK(p.id && *p.id == 7 && p.name == "rex" && p.photoUrls.size() == 2 && p.photoUrls[1] == "http://x/2");
  CHECK(p.category && p.category->name && *p.category->name == "dogs" && p.tags && p.tags->size() == 1 && *(*p.tags)[0].name == "good");
  CHECK(p.status && *p.status == PetStatus::PENDING);
  CHECK(om.writeValueAsString(p) == doc);  // field order, number formatting and escaping as the serialiser rules say

  // escapes are decoded on the way in and re-applied on the way out
  Pet q = om.readValue<Pet>("{ \"name\" : \"a\\u00e9\\n\\\"\" , \"photoUrls\" : [] }");
  CHECK(q.name == "a\xc3\xa9\n\"" && q.photoUrls.empty() && !q.id && !q.tags);
  ObjectMapper keep_empty(-1, PJ_INCLUDE_NON_NULL);
  CHECK(keep_empty.writeValueAsString(q) == "{\"name\":\"a\xc3\xa9\\n\\\"\",\"photoUrls\":[]}");

  // validation failures surface as exceptions with kind and byte offset
  try { om.readValue<Pet>("{\"id\":1,\"photoUrls\":[]}"); CHECK(false); }
  catch (const SerdeException& e) { CHECK(e.kind == PJ_E_REQUIRED && e.offset == 22); }
  try { om.readValue<Pet>("{\"name\":\"a\",\"photoUrls\":[],\"status\":\"lost\"}"); CHECK(false); }
  catch (const SerdeException& e) { CHECK(e.kind == PJ_E_ENUM && e.offset == 36); }
  try { om.readValue<Order>("{\"quantity\":\"3\"}"); CHECK(false); }
  catch (const SerdeException& e) { CHECK(e.kind == PJ_E_TYPE && e.offset == 12); }

  // a batch, one record per line
  const std::string batch = "{\"id\":1,\"petId\":7,\"quantity\":2,\"shipDate\":\"2024-02-29T23:59:59.5+05:30\",\"status\":\"approved\",\"complete\":true}\n"
                            "{\"id\":2}\n";
  std::vector<Order> orders = om.readValues<Order>(reinterpret_cast<const uint8_t*>(batch.data()), batch.size());
  CHECK(orders.size() == 2 && orders[0].shipDate && orders[0].shipDate->nano == 500000000 && orders[0].shipDate->offsetSeconds == 19800);
  CHECK(*orders[0].complete && !orders[1].petId);
  CHECK(om.writeValuesAsString(orders) == batch);

  User u;
  u.id = 5; u.username = "bob"; u.userStatus = 1;
  CHECK(om.writeValueAsString(u) == "{\"id\":5,\"username\":\"bob\",\"userStatus\":1}");
  CHECK(om.writeValuesAsString(std::vector<User>{u, u}, PJ_FRAMING_ARRAY) ==
        "[{\"id\":5,\"username\":\"bob\",\"userStatus\":1},{\"id\":5,\"username\":\"bob\",\"userStatus\":1}]");
  std::puts("object mapper ok");
  return 0;
}
