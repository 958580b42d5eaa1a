"""Schema compiler: OpenAPI / Swagger model definitions -> the compile-time model tables of the kernels.

    python -m "micronaut3-bug_b200.schemac" petstore.json            # prints csrc/pj_schema_models.inc
    python -m "micronaut3-bug_b200.schemac" petstore.json --write    # rewrites it in place
    python -m "micronaut3-bug_b200.schemac" swagger.yml --check      # lists what the tables cannot express yet

The reference feeds its specs to the OpenAPI generator, which emits the model classes that Micronaut Serde then
(de)serialises (build.gradle:43-62 of altro3/micronaut3-bug); here the same definitions become `CObj<>` / `CEnum<>`
tables (kind, column, counter slot and child of every property, in specification order, with the required set),
on which the tokenisers and writers are instantiated. What a definition uses beyond the supported subset is reported
by --check instead of being silently dropped.

Supported: objects of properties whose types are integer (int64 / int32), boolean, string, string with `enum`,
string of format date-time, a `$ref` to a flat object (scalar properties only), arrays of strings and arrays of
`$ref`s to flat objects; `required`. Not expressible yet (reported): `number` (doubles), `allOf` / `oneOf` / `anyOf`,
`discriminator`, `default`, `minimum` / `maximum` and the other validation keywords, `additionalProperties`, nested
arrays, arrays of scalars other than strings, `$ref`s that are mere aliases of scalars.
"""
from __future__ import annotations

import json
import os
import re
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(PKG, "csrc", "pj_schema_models.inc")

# How the Petstore models map onto the column ids of include/petjson.h and the counter slots of csrc/pj_schema.h:
# per model its object id, PJ_TYPE_*, column prefix and, per property, the token its columns are named with
# (an embedded object or list element gets a prefix of its own). Everything else comes from the specification.
LAYOUT = {
    "Pet": {"obj": "OBJ_PET", "type": "PJ_TYPE_PET", "prefix": "PET", "where": "petstore.json:872-922, required name + photoUrls (:873-876)",
            "props": {"id": "ID", "category": "CAT", "name": "NAME", "photoUrls": "PHOTO", "tags": ("TAGS", "TAG"), "status": "STATUS"}},
    "Category": {"obj": "OBJ_CATEGORY", "type": "0", "prefix": "PET_CAT", "where": "petstore.json:858-871", "props": {"id": "ID", "name": "NAME"}},
    "Tag": {"obj": "OBJ_TAG", "type": "0", "prefix": "PET_TAG", "where": "petstore.json:923-936", "props": {"id": "ID", "name": "NAME"}},
    "Order": {"obj": "OBJ_ORDER", "type": "PJ_TYPE_ORDER", "prefix": "ORD", "where": "petstore.json:937-971",
              "props": {"id": "ID", "petId": "PET_ID", "quantity": "QUANTITY", "shipDate": "SHIP_EPOCH", "status": "STATUS", "complete": "COMPLETE"}},
    "User": {"obj": "OBJ_USER", "type": "PJ_TYPE_USER", "prefix": "USR", "where": "petstore.json:824-857", "indexed_string_slots": "SLOT_USR_STR0",
             "props": {"id": "ID", "username": "USERNAME", "firstName": "FIRSTNAME", "lastName": "LASTNAME", "email": "EMAIL", "password": "PASSWORD",
                       "phone": "PHONE", "userStatus": "STATUS"}},
}
ORDER = ["Pet", "Category", "Tag", "Order", "User"]  # the order of ObjId
ENUM_WHERE = {("Pet", "status"): "petstore.json:912-916", ("Order", "status"): ":958-962"}

UNSUPPORTED_KEYS = ("allOf", "oneOf", "anyOf", "not", "discriminator", "additionalProperties", "patternProperties")
VALIDATION_KEYS = ("minimum", "maximum", "exclusiveMinimum", "exclusiveMaximum", "multipleOf", "minLength", "maxLength", "pattern",
                   "minItems", "maxItems", "uniqueItems", "default", "const", "nullable")


def load_spec(path: str) -> dict:
    with open(path) as f:
        text = f.read()
    if path.endswith((".yml", ".yaml")):
        import yaml

        return yaml.safe_load(text)
    return json.loads(text)


def definitions(spec: dict) -> dict:
    """Swagger 2.0 `definitions` or OpenAPI 3 `components.schemas`."""
    if "definitions" in spec:
        return spec["definitions"]
    return spec.get("components", {}).get("schemas", {})


def ref_name(ref: str) -> str:
    return ref.rsplit("/", 1)[-1]


def classify(prop: dict, defs: dict, problems: list, where: str, flat: bool) -> tuple[str, str | None]:
    """(kind, child definition) of one property; appends what cannot be expressed to `problems`."""
    for k in UNSUPPORTED_KEYS:
        if k in prop:
            problems.append(f"{where}: `{k}` is not expressible")
    for k in VALIDATION_KEYS:
        if k in prop:
            problems.append(f"{where}: `{k}` ({prop[k]!r}) is not validated or applied")
    if "$ref" in prop:
        name = ref_name(prop["$ref"])
        target = defs.get(name, {})
        if target.get("type") != "object" and "properties" not in target:
            problems.append(f"{where}: `$ref` to `{name}`, which is not an object of properties (an alias or a composition)")
            return "?", None
        if flat:
            problems.append(f"{where}: an object inside an embedded object or list element (only one level is flat)")
        return "K_OBJ", name
    t, fmt = prop.get("type"), prop.get("format")
    if t == "integer":
        return ("K_I32" if fmt == "int32" else "K_I64"), None
    if t == "boolean":
        return "K_BOOL", None
    if t == "string":
        if "enum" in prop:
            return "K_ENUM", None
        if fmt == "date-time":
            return "K_DATETIME", None
        if fmt not in (None, "password", "byte", "binary", "email", "uuid", "uri", "hostname"):
            problems.append(f"{where}: string format `{fmt}` is kept as plain text")
        return "K_STR", None
    if t == "array":
        items = prop.get("items", {})
        if flat:
            problems.append(f"{where}: a list inside an embedded object or list element")
        if "$ref" in items:
            name = ref_name(items["$ref"])
            target = defs.get(name, {})
            if target.get("type") != "object" and "properties" not in target:
                problems.append(f"{where}: list of `{name}`, which is not an object of properties")
                return "?", None
            return "K_LIST_OBJ", name
        if items.get("type") == "string" and "enum" not in items:
            return "K_LIST_STR", None
        problems.append(f"{where}: list of `{items.get('type', items)}` (only lists of strings and of flat objects)")
        return "?", None
    if t == "number":
        problems.append(f"{where}: `number` (double precision) has no kind yet")
        return "?", None
    problems.append(f"{where}: type `{t}` is not expressible")
    return "?", None


def check(defs: dict) -> list[str]:
    """Everything in `defs` that the model tables cannot express."""
    problems: list[str] = []
    for name, d in defs.items():
        for k in UNSUPPORTED_KEYS:
            if k in d:
                problems.append(f"{name}: `{k}` is not expressible")
        if "$ref" in d and len(d) <= 2:
            problems.append(f"{name}: an alias of `{ref_name(d['$ref'])}`")
            continue
        props = d.get("properties")
        if props is None:
            if d.get("type") != "object":
                problems.append(f"{name}: not an object of properties (type `{d.get('type')}`)")
            continue
        if len(props) > 8:
            problems.append(f"{name}: {len(props)} properties (tables hold 8 per object)")
        for pname, p in props.items():
            if len(pname) > 13:
                problems.append(f"{name}.{pname}: property names longer than 13 bytes are not matched by the word compare")
            classify(p, defs, problems, f"{name}.{pname}", flat=False)
    return problems


def emit(defs: dict, layout: dict = LAYOUT, order: list[str] = ORDER) -> str:
    """The text of csrc/pj_schema_models.inc for the laid-out models."""
    problems: list[str] = []
    enums: list[tuple[str, str, list[str]]] = []
    out = ["/* GENERATED by `python -m micronaut3-bug_b200.schemac` from the OpenAPI definitions; do not edit: change the",
           " * specification or the layout table of schemac.py and regenerate. One CObj<> per object in ObjId order: every property",
           " * in specification order with its kind, column, counter slot and child; CEnum<> holds the literals of the enums. */"]
    for name in order:
        d, lay = defs[name], layout[name]
        props = d["properties"]
        required = d.get("required", [])
        keys = list(props)
        req_bits = " | ".join(f"(1 << {keys.index(r)})" for r in required) if required else "0"
        out.append(f"/* {name} — {lay['where']} */")
        out.append(f"template <> struct CObj<{lay['obj']}> {{")
        out.append(f"  static constexpr int N = {len(keys)}, present_col = PJ_COL_{lay['prefix']}_PRESENT, required = {req_bits}, type = {lay['type']};")
        out.append("  static constexpr CF f[N] = {")
        nstr = 0
        flat = lay["type"] == "0"
        for pname in keys:
            kind, child = classify(props[pname], defs, problems, f"{name}.{pname}", flat)
            tok = lay["props"][pname]
            col = f"PJ_COL_{lay['prefix']}_"
            if kind in ("K_I64", "K_I32", "K_BOOL", "K_DATETIME"):
                args = f"{kind}, {col}{tok}"
            elif kind == "K_ENUM":
                enums.append((name, pname, props[pname]["enum"]))
                args = f"{kind}, {col}{tok}, 0, {len(enums) - 1}"
            elif kind == "K_STR":
                slot = f"{lay['indexed_string_slots']} + {nstr}" if "indexed_string_slots" in lay else f"SLOT_{lay['prefix']}_{tok}"
                nstr += 1
                args = f"{kind}, {col}{tok}_OFF, {slot}"
            elif kind == "K_OBJ":
                args = f"{kind}, 0, 0, {layout[child]['obj']}"
            elif kind == "K_LIST_STR":
                args = f"{kind}, {col}{tok}_OFF, SLOT_{lay['prefix']}_{tok}_CNT"
            elif kind == "K_LIST_OBJ":
                list_tok, elem_tok = tok
                args = f"{kind}, {col}{list_tok}_OFF, SLOT_{lay['prefix']}_{elem_tok}_CNT, {layout[child]['obj']}"
            else:
                raise SystemExit(f"{name}.{pname}: not expressible: " + "; ".join(problems))
            out.append(f"      cf(\"{pname}\", {args}),")
        out[-1] = out[-1].rstrip(",") + "};"
        out.append("};")
    if problems:
        raise SystemExit("not expressible: " + "; ".join(problems))
    out.append("/* enum literals: " + ", ".join(f"{k} {n}.{p} ({ENUM_WHERE.get((n, p), '')})" for k, (n, p, _) in enumerate(enums)) + " */")
    for k, (_, _, lits) in enumerate(enums):
        body = ", ".join(f'cf("{lit}", K_ENUM, 0)' for lit in lits)
        out.append(f"template <> struct CEnum<{k}> {{ static constexpr int N = {len(lits)}; static constexpr CF lit[N] = {{{body}}}; }};")
    return "\n".join(out) + "\n"


def main(argv: list[str]) -> int:
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    defs = definitions(load_spec(argv[0]))
    if "--check" in argv:
        problems = check(defs)
        for p in problems:
            print(p)
        print(f"{len(defs)} definitions, {len(problems)} constructs not expressible yet")
        return 0
    text = emit(defs)
    if "--write" in argv:
        with open(OUT, "w") as f:
            f.write(text)
        print(OUT)
    else:
        sys.stdout.write(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main(sys.argv[1:]))
