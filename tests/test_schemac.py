"""The schema compiler (micronaut3-bug_b200/schemac.py): OpenAPI definitions -> the kernels' compile-time model tables."""
import importlib
import os

import pytest

from pj_testlib import ROOT

schemac = importlib.import_module("micronaut3-bug_b200.schemac")

I64 = {"type": "integer", "format": "int64"}
I32 = {"type": "integer", "format": "int32"}
STR = {"type": "string"}
# The five definitions of the Petstore specification, restated: names, order, types, required sets and literals are
# what the model tables must carry (petstore.json:823-972 of the reference project holds the same facts).
PETSTORE = {
    "User": {"type": "object", "properties": {"id": I64, "username": STR, "firstName": STR, "lastName": STR, "email": STR, "password": STR,
                                              "phone": STR, "userStatus": dict(I32, description="User Status")}},
    "Category": {"type": "object", "properties": {"id": I64, "name": STR}},
    "Pet": {"type": "object", "required": ["name", "photoUrls"],
            "properties": {"id": I64, "category": {"$ref": "#/definitions/Category"}, "name": dict(STR, example="doggie"),
                           "photoUrls": {"type": "array", "items": STR}, "tags": {"type": "array", "items": {"$ref": "#/definitions/Tag"}},
                           "status": dict(STR, enum=["available", "pending", "sold"])}},
    "Tag": {"type": "object", "properties": {"id": I64, "name": STR}},
    "Order": {"type": "object", "properties": {"id": I64, "petId": I64, "quantity": I32, "shipDate": {"type": "string", "format": "date-time"},
                                               "status": dict(STR, enum=["placed", "approved", "delivered"]), "complete": {"type": "boolean"}}},
}


def committed() -> str:
    with open(os.path.join(ROOT, "micronaut3-bug_b200", "csrc", "pj_schema_models.inc")) as f:
        return f.read()


def test_the_committed_tables_are_the_compilers_output():
    assert schemac.emit(PETSTORE) == committed()
    assert schemac.check(PETSTORE) == []


@pytest.mark.skipif(not os.path.exists("/root/reference/petstore.json"), reason="the reference checkout is not on this machine")
def test_the_reference_specification_compiles_to_the_same_tables():
    defs = schemac.definitions(schemac.load_spec("/root/reference/petstore.json"))
    assert schemac.emit(defs) == committed()


def test_what_the_tables_cannot_express_is_reported():
    defs = {
        "Base": {"type": "object", "discriminator": {"propertyName": "_o"}, "required": ["_o"], "properties": {"_o": STR, "up": {"type": "boolean"}}},
        "Alias": {"$ref": "#/components/schemas/Base"},
        "Derived": {"allOf": [{"$ref": "#/components/schemas/Alias"}, {"type": "object", "properties": {"field": dict(STR, enum=["a", "b"])}}]},
        "Page": {"type": "object", "properties": {"page": dict(I64, default=0, minimum=0), "ratio": {"type": "number"}, "grid": {"type": "array", "items": {"type": "array", "items": STR}},
                                                  "aVeryLongPropertyName": STR, "sort": {"type": "array", "items": {"$ref": "#/components/schemas/Alias"}}}},
    }
    got = "\n".join(schemac.check(defs))
    for needle in ("Base: `discriminator`", "Alias: an alias of `Base`", "Derived: `allOf`", "Page.page: `default`", "Page.page: `minimum`",
                   "Page.ratio: `number`", "Page.grid: list of", "Page.aVeryLongPropertyName: property names longer", "Page.sort: list of `Alias`"):
        assert needle in got, needle
    with pytest.raises(SystemExit):
        schemac.emit({**PETSTORE, "Pet": {"type": "object", "properties": {**PETSTORE["Pet"]["properties"], "id": {"type": "number"}}}})


@pytest.mark.skipif(not os.path.exists("/root/reference/swagger.yml"), reason="the reference checkout is not on this machine")
def test_the_generated_model_set_of_the_reference_is_listed_as_work_to_do():
    defs = schemac.definitions(schemac.load_spec("/root/reference/swagger.yml"))
    problems = schemac.check(defs)
    assert any("allOf" in p for p in problems) and any("discriminator" in p for p in problems)
    assert any("`minimum`" in p for p in problems) and any("`default`" in p for p in problems)
