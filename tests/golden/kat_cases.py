"""Hand-written known-answer cases for the parse / validate rules (R1-R12 of include/petjson.h).

Every expectation here was derived by hand from the rules, not by running any implementation:
offsets are written as "position of this token in the input", dates are computed with Python's
datetime. The reference project has no test vectors for this path, so these take their place for
pinning the CPU checker; the same cases are then run through the CUDA path.

CASE = (name, schema, framing, input bytes, expected)
expected = list with one entry per record: a dict of decoded values, or (KIND, offset).
For array framing an optional trailing element {"doc": (KIND, offset)} describes the document fault.
"""
from datetime import datetime, timedelta, timezone


def at(s: bytes, tok: bytes, nth: int = 0) -> int:
    """Offset of the nth occurrence of tok in s."""
    i = -1
    for _ in range(nth + 1):
        i = s.index(tok, i + 1)
    return i


def epoch(y, mo, d, h, mi, s, off_s=0):
    return int(datetime(y, mo, d, h, mi, s, tzinfo=timezone(timedelta(seconds=off_s))).timestamp())


CASES = []


def case(name, schema, data, expected, framing="ndjson"):
    CASES.append((name, schema, framing, data, expected))


def err1(name, schema, data, kind, off, framing="ndjson"):
    """A single-record input that must fail with (kind, off)."""
    case(name, schema, data, [(kind, off)], framing)


MIN = b'"name":"a","photoUrls":[]'  # the two required Pet properties
MIN_D = {"name": "a", "photoUrls": []}

# ---- accepted records ----------------------------------------------------------------------------
case("pet minimal", "pet", b'{' + MIN + b'}\n', [MIN_D])
case("pet full", "pet",
     b'{"id":12,"category":{"id":3,"name":"dogs"},"name":"rex","photoUrls":["http://x/y","z"],'
     b'"tags":[{"id":1,"name":"t1"},{"id":2,"name":"t2"}],"status":"pending"}\n',
     [{"id": 12, "category": {"id": 3, "name": "dogs"}, "name": "rex", "photoUrls": ["http://x/y", "z"],
       "tags": [{"id": 1, "name": "t1"}, {"id": 2, "name": "t2"}], "status": "pending"}])
case("pet any key order + unknown keys", "pet",
     b'{"status":"sold","x":{"a":[1,2.5e-3,{"b":null}],"c":"d"},"photoUrls":["p"],"y":[],"tags":[],"name":"n","z":-0.0,"id":7}\n',
     [{"id": 7, "name": "n", "photoUrls": ["p"], "tags": [], "status": "sold"}])
case("pet whitespace and CRLF", "pet",
     b' \t{ "id" :\t1 , "name"\r: "a" ,"photoUrls" : [ "u" , "v" ] } \r\n',
     [{"id": 1, "name": "a", "photoUrls": ["u", "v"]}])
case("pet nulls are absent", "pet",
     b'{"id":null,"category":null,"name":"a","photoUrls":[],"tags":null,"status":null}\n', [MIN_D])
case("pet empty nested objects", "pet",
     b'{"category":{},"name":"a","photoUrls":[],"tags":[{},{"name":null,"id":null}]}\n',
     [{"category": {}, "name": "a", "photoUrls": [], "tags": [{}, {}]}])
case("pet repeated keys: last wins", "pet",
     b'{"name":"first","photoUrls":["x","y"],"name":"b","photoUrls":[],"id":1,"id":2,'
     b'"tags":[{"id":1,"name":"q"}],"tags":[{"name":"r","name":"s"}],"category":{"id":1,"name":"c"},"category":{"name":"d"}}\n',
     [{"id": 2, "category": {"name": "d"}, "name": "b", "photoUrls": [], "tags": [{"name": "s"}]}])
case("pet repeated key then null", "pet",
     b'{"name":"a","photoUrls":[],"status":"sold","status":null,"id":5,"id":null}\n', [MIN_D])
case("pet escapes", "pet",
     b'{"name":"\\u0041\\n\\"\\\\\\/\\b\\f\\r\\t\\u00e9\\u20AC\\ud83d\\ude00","photoUrls":["\\u0000"]}\n',
     [{"name": 'A\n"\\/\b\f\r\t\u00e9\u20ac\U0001F600', "photoUrls": ["\x00"]}])
case("pet raw utf-8", "pet", '{"name":"é€😀\U0010FFFF","photoUrls":[]}\n'.encode(),
     [{"name": "é€😀\U0010FFFF", "photoUrls": []}])
case("pet escaped key and enum", "pet", b'{"\\u006eame":"a","photoUrls":[],"st\\u0061tus":"s\\u006fld"}\n',
     [{"name": "a", "photoUrls": [], "status": "sold"}])
case("pet integer edges", "pet",
     b'{"id":9223372036854775807,' + MIN + b'}\n{"id":-9223372036854775808,' + MIN + b'}\n{"id":-0,' + MIN + b'}\n{"id":0,' + MIN + b'}\n',
     [dict(MIN_D, id=9223372036854775807), dict(MIN_D, id=-9223372036854775808), dict(MIN_D, id=0), dict(MIN_D, id=0)])
case("blank lines skipped, last line unterminated", "pet",
     b'\n  \n{' + MIN + b'}\n\r\n\t\n{"id":1,' + MIN + b'}', [MIN_D, dict(MIN_D, id=1)])
case("empty input", "pet", b'', [])
case("only blank lines", "pet", b'\n\n \r\n', [])
case("skipped values: 64 nested arrays are allowed", "pet", b'{"x":' + b'[' * 64 + b']' * 64 + b',' + MIN + b'}\n', [MIN_D])
case("empty strings", "pet", b'{"name":"","photoUrls":["",""],"tags":[{"name":""}],"category":{"name":""}}\n',
     [{"category": {"name": ""}, "name": "", "photoUrls": ["", ""], "tags": [{"name": ""}]}])

# ---- syntax ------------------------------------------------------------------------------------
s = b'{"id":01,' + MIN + b'}\n'; err1("leading zero", "pet", s, "SYNTAX", at(s, b'01') + 1)
s = b'{"id":+1,' + MIN + b'}\n'; err1("leading plus", "pet", s, "SYNTAX", at(s, b'+'))
s = b'{"id":1.,' + MIN + b'}\n'; err1("fraction without digits", "pet", s, "SYNTAX", at(s, b'.,') + 1)
s = b'{"id":-,' + MIN + b'}\n'; err1("minus without digits", "pet", s, "SYNTAX", at(s, b'-,') + 1)
s = b'{"id":1e,' + MIN + b'}\n'; err1("exponent without digits", "pet", s, "SYNTAX", at(s, b'e,') + 1)
s = b'{"id":.5,' + MIN + b'}\n'; err1("fraction without integer part", "pet", s, "SYNTAX", at(s, b'.5'))
s = b'{"id":NaN,' + MIN + b'}\n'; err1("NaN", "pet", s, "SYNTAX", at(s, b'NaN'))
s = b'{/*c*/' + MIN + b'}\n'; err1("block comment", "pet", s, "SYNTAX", 1)
s = b'{' + MIN + b'} // c\n'; err1("line comment after record", "pet", s, "SYNTAX", at(s, b'//'))
s = b'# c\n'; err1("hash comment", "pet", s, "SYNTAX", 0)
s = b"{'name':'a'}\n"; err1("single quotes", "pet", s, "SYNTAX", 1)
s = b'{' + MIN + b',}\n'; err1("trailing comma in object", "pet", s, "SYNTAX", at(s, b',}') + 1)
s = b'{"name":"a","photoUrls":["x",]}\n'; err1("trailing comma in list", "pet", s, "SYNTAX", at(s, b',]') + 1)
s = b'{"name":"a","photoUrls":["x" "y"]}\n'; err1("missing comma in list", "pet", s, "SYNTAX", at(s, b'"y"'))
s = b'{"name" "a"}\n'; err1("missing colon", "pet", s, "SYNTAX", at(s, b'"a"'))
s = b'{"name":"a" "photoUrls":[]}\n'; err1("missing comma in object", "pet", s, "SYNTAX", at(s, b'"photoUrls"'))
s = b'{name:"a"}\n'; err1("unquoted key", "pet", s, "SYNTAX", 1)
s = b'{' + MIN + b'} x\n'; err1("trailing garbage", "pet", s, "SYNTAX", at(s, b' x') + 1)
s = b'{' + MIN + b'}{' + MIN + b'}\n'; err1("two objects on a line", "pet", s, "SYNTAX", at(s, b'}{') + 1)
s = b'x\n'; err1("not json", "pet", s, "SYNTAX", 0)
s = b'{"name":"a","photoUrls":[],"x":tru}\n'; err1("bad literal", "pet", s, "SYNTAX", at(s, b'tru}') + 3)
s = b'{"name":"a","photoUrls":[],"x":nulL}\n'; err1("bad literal case", "pet", s, "SYNTAX", at(s, b'nulL') + 3)
s = b'{"name":"a","photoUrls":[],"x":[1 2]}\n'; err1("skipped value: missing comma", "pet", s, "SYNTAX", at(s, b'1 2') + 2)
s = b'{"name":"a","photoUrls":[],"x":{"k" 1}}\n'; err1("skipped value: missing colon", "pet", s, "SYNTAX", at(s, b'"k" 1') + 4)
s = b'{"name":"a","photoUrls":[],"x":{"k":1,}}\n'; err1("skipped value: trailing comma", "pet", s, "SYNTAX", at(s, b',}') + 1)
s = b'{"name":"a","photoUrls":[],"x":[}\n'; err1("skipped value: mismatched bracket", "pet", s, "SYNTAX", at(s, b'[}') + 1)
s = '{"name":"a","photoUrls":[],\u00e9:1}\n'.encode(); err1("non-ascii outside a string", "pet", s, "SYNTAX", at(s, '\u00e9'.encode()))

# ---- end of record -----------------------------------------------------------------------------
for name, body in [("inside a string", b'{"id":1,"name":"ab'), ("after a comma", b'{"id":1,'), ("after a colon", b'{"id":'),
                   ("after a number", b'{"id":12'), ("inside a literal", b'{"name":"a","photoUrls":[],"x":tr'),
                   ("inside an escape", b'{"name":"a\\'), ("inside \\u", b'{"name":"a\\u00'), ("after the brace", b'{'),
                   ("inside a list", b'{"name":"a","photoUrls":["x"'), ("after a high surrogate", b'{"name":"\\ud83d'),
                   ("inside a utf-8 sequence", b'{"name":"\xe2\x82'), ("after minus", b'{"id":-'), ("after a key", b'{"id"')]:
    err1("record ends " + name, "pet", body + b'\n', "EOF", len(body))
    err1("input ends " + name, "pet", body, "EOF", len(body))

# ---- strings --------------------------------------------------------------------------------------
s = b'{"name":"a\tb","photoUrls":[]}\n'; err1("raw tab in string", "pet", s, "CTRL_CHAR", at(s, b'\t'))
s = b'{"name":"a\x00b","photoUrls":[]}\n'; err1("raw NUL in string", "pet", s, "CTRL_CHAR", at(s, b'\x00'))
s = b'{"name":"a\rb","photoUrls":[]}\n'; err1("raw CR in string", "pet", s, "CTRL_CHAR", at(s, b'\r'))
s = b'{"name":"\\x41","photoUrls":[]}\n'; err1("unknown escape", "pet", s, "BAD_ESCAPE", at(s, b'\\x') + 1)
s = b'{"name":"\\u12G4","photoUrls":[]}\n'; err1("bad hex digit", "pet", s, "BAD_ESCAPE", at(s, b'G'))
s = b'{"name":"\\ude00","photoUrls":[]}\n'; err1("lone low surrogate", "pet", s, "BAD_SURROGATE", at(s, b'\\ude00'))
s = b'{"name":"\\ud83d","photoUrls":[]}\n'; err1("high surrogate then quote", "pet", s, "BAD_SURROGATE", at(s, b'\\ud83d'))
s = b'{"name":"\\ud83d\\u0041","photoUrls":[]}\n'; err1("high surrogate then BMP", "pet", s, "BAD_SURROGATE", at(s, b'\\ud83d'))
s = b'{"name":"\\ud83d\\n","photoUrls":[]}\n'; err1("high surrogate then \\n", "pet", s, "BAD_SURROGATE", at(s, b'\\ud83d'))
s = b'{"name":"\\ud83d\\ud83d","photoUrls":[]}\n'; err1("two high surrogates", "pet", s, "BAD_SURROGATE", at(s, b'\\ud83d'))
s = b'{"name":"\\ud83d\\uZZZZ","photoUrls":[]}\n'; err1("high surrogate then bad hex", "pet", s, "BAD_ESCAPE", at(s, b'ZZZZ'))
for name, bad in [("overlong C0", b'\xc0\x80'), ("overlong E0", b'\xe0\x80\x80'), ("surrogate ED A0", b'\xed\xa0\x80'),
                  ("lead F5", b'\xf5\x80\x80\x80'), ("above U+10FFFF", b'\xf4\x90\x80\x80'), ("lone continuation", b'\x80'),
                  ("truncated sequence", b'\xe2\x82'), ("overlong F0", b'\xf0\x8f\x80\x80'), ("lead FF", b'\xff')]:
    s = b'{"name":"ok' + bad + b'","photoUrls":[]}\n'
    err1("utf-8: " + name, "pet", s, "UTF8", at(s, bad))
s = b'{"\xc0\x80":1,' + MIN + b'}\n'; err1("utf-8 in a key", "pet", s, "UTF8", 2)
s = b'{"x":"\xff",' + MIN + b'}\n'; err1("utf-8 in a skipped value", "pet", s, "UTF8", at(s, b'\xff'))

# ---- types ------------------------------------------------------------------------------------
s = b'[1,2]\n'; err1("record is an array", "pet", s, "TYPE", 0)
s = b'"str"\n'; err1("record is a string", "pet", s, "TYPE", 0)
s = b'null\n'; err1("record is null", "pet", s, "TYPE", 0)
s = b'  12\n'; err1("record is a number", "pet", s, "TYPE", 2)
for name, val in [("string", b'"1"'), ("bool", b'true'), ("object", b'{}'), ("array", b'[1]')]:
    s = b'{"id":' + val + b',' + MIN + b'}\n'; err1("id is " + name, "pet", s, "TYPE", at(s, b'"id":') + 5)
s = b'{"id":1.5,' + MIN + b'}\n'; err1("id has a fraction", "pet", s, "TYPE", at(s, b'1.5'))
s = b'{"id":1e3,' + MIN + b'}\n'; err1("id has an exponent", "pet", s, "TYPE", at(s, b'1e3'))
s = b'{"id":1.0,' + MIN + b'}\n'; err1("id is 1.0", "pet", s, "TYPE", at(s, b'1.0'))
s = b'{"name":1,"photoUrls":[]}\n'; err1("name is a number", "pet", s, "TYPE", at(s, b':1') + 1)
s = b'{"name":true,"photoUrls":[]}\n'; err1("name is a bool", "pet", s, "TYPE", at(s, b'true'))
s = b'{"name":"a","photoUrls":"x"}\n'; err1("photoUrls is a string", "pet", s, "TYPE", at(s, b'"x"'))
s = b'{"name":"a","photoUrls":{}}\n'; err1("photoUrls is an object", "pet", s, "TYPE", at(s, b'{}'))
s = b'{"name":"a","photoUrls":[1]}\n'; err1("photoUrls item is a number", "pet", s, "TYPE", at(s, b'[1]') + 1)
s = b'{"name":"a","photoUrls":[null]}\n'; err1("photoUrls item is null", "pet", s, "TYPE", at(s, b'null'))
s = b'{"name":"a","photoUrls":[],"tags":[1]}\n'; err1("tag is a number", "pet", s, "TYPE", at(s, b'[1]') + 1)
s = b'{"name":"a","photoUrls":[],"tags":[null]}\n'; err1("tag is null", "pet", s, "TYPE", at(s, b'null'))
s = b'{"name":"a","photoUrls":[],"tags":[{"id":"x"}]}\n'; err1("tag id is a string", "pet", s, "TYPE", at(s, b'"x"'))
s = b'{"name":"a","photoUrls":[],"tags":{}}\n'; err1("tags is an object", "pet", s, "TYPE", at(s, b'{}'))
s = b'{"name":"a","photoUrls":[],"category":[]}\n'; err1("category is an array", "pet", s, "TYPE", at(s, b'[]', 1))
s = b'{"name":"a","photoUrls":[],"category":{"name":5}}\n'; err1("category name is a number", "pet", s, "TYPE", at(s, b'5'))
s = b'{"name":"a","photoUrls":[],"status":1}\n'; err1("status is a number", "pet", s, "TYPE", at(s, b':1') + 1)
s = b'{"name":"a","photoUrls":[@]}\n'; err1("list item starts no value", "pet", s, "SYNTAX", at(s, b'@'))
s = b'{"name":@,"photoUrls":[]}\n'; err1("value starts no value", "pet", s, "SYNTAX", at(s, b'@'))

# ---- ranges, enums, required -------------------------------------------------------------------
s = b'{"id":9223372036854775808,' + MIN + b'}\n'; err1("int64 max + 1", "pet", s, "NUM_RANGE", at(s, b'922'))
s = b'{"id":-9223372036854775809,' + MIN + b'}\n'; err1("int64 min - 1", "pet", s, "NUM_RANGE", at(s, b'-922'))
s = b'{"id":18446744073709551616,' + MIN + b'}\n'; err1("2^64", "pet", s, "NUM_RANGE", at(s, b'184'))
s = b'{"id":' + b'9' * 40 + b',' + MIN + b'}\n'; err1("40 digits", "pet", s, "NUM_RANGE", at(s, b'999'))
s = b'{"name":"a","photoUrls":[],"status":"unknown"}\n'; err1("unknown enum literal", "pet", s, "ENUM", at(s, b'"unknown"'))
s = b'{"name":"a","photoUrls":[],"status":"Sold"}\n'; err1("enum is case sensitive", "pet", s, "ENUM", at(s, b'"Sold"'))
s = b'{"name":"a","photoUrls":[],"status":""}\n'; err1("empty enum literal", "pet", s, "ENUM", at(s, b'""'))
s = b'{"name":"a","photoUrls":[],"status":"availablex"}\n'; err1("enum with a suffix", "pet", s, "ENUM", at(s, b'"availablex"'))
s = b'{"name":"a","photoUrls":[],"status":"placed"}\n'; err1("Order literal on a Pet", "pet", s, "ENUM", at(s, b'"placed"'))
s = b'{"photoUrls":[]}\n'; err1("name missing", "pet", s, "REQUIRED", len(s) - 2)
s = b'{"name":"a"}\n'; err1("photoUrls missing", "pet", s, "REQUIRED", len(s) - 2)
s = b'{"name":null,"photoUrls":[]}\n'; err1("name null", "pet", s, "REQUIRED", len(s) - 2)
s = b'{}\n'; err1("empty object", "pet", s, "REQUIRED", 1)
s = b'{"name":"a","photoUrls":[],"name":null } x\n'; err1("required beats trailing garbage", "pet", s, "REQUIRED", at(s, b'} x'))
s = b'{"x":' + b'[' * 65 + b']' * 65 + b',' + MIN + b'}\n'; err1("65 nested arrays", "pet", s, "DEPTH", at(s, b'[') + 64)
s = b'{"x":' + b'{"k":' * 65 + b'1' + b'}' * 65 + b',' + MIN + b'}\n'; err1("65 nested objects", "pet", s, "DEPTH", at(s, b'{"k":') + 5 * 64)
# first failure in reading order wins
s = b'{"id":"x","status":"bad"}\n'; err1("first failure wins", "pet", s, "TYPE", at(s, b'"x"'))
s = b'{"status":"b\\qd","id":"x"}\n'; err1("lexical failure inside an enum value", "pet", s, "BAD_ESCAPE", at(s, b'\\q') + 1)

# ---- Order ---------------------------------------------------------------------------------------
case("order full", "order",
     b'{"id":1,"petId":2,"quantity":3,"shipDate":"2024-02-29T23:59:59.5+05:30","status":"approved","complete":true}\n',
     [{"id": 1, "petId": 2, "quantity": 3, "shipDate": (epoch(2024, 2, 29, 23, 59, 59, 19800), 500000000, 19800),
       "status": "approved", "complete": True}])
case("order dates", "order",
     b'{"shipDate":"1970-01-01T00:00:00Z"}\n{"shipDate":"1969-12-31T23:59:59.999999999-00:01"}\n'
     b'{"shipDate":"9999-12-31T23:59:59+00:00"}\n{"shipDate":"0000-01-01T00:00:00.000000001Z"}\n{"shipDate":"2000-02-29T12:00:00-23:59"}\n',
     [{"shipDate": (0, 0, 0)}, {"shipDate": (-1 + 60, 999999999, -60)},
      {"shipDate": (epoch(9999, 12, 31, 23, 59, 59), 0, 0)}, {"shipDate": (-62167219200, 1, 0)},
      {"shipDate": (epoch(2000, 2, 29, 12, 0, 0, -86340), 0, -86340)}])
case("order empty and nulls", "order", b'{}\n{"complete":null,"quantity":null,"shipDate":null}\n{"complete":false,"quantity":-2147483648}\n',
     [{}, {}, {"complete": False, "quantity": -2147483648}])
for name, text in [("month 13", b'2020-13-01T00:00:00Z'), ("feb 29 in 2021", b'2021-02-29T00:00:00Z'), ("feb 29 in 1900", b'1900-02-29T00:00:00Z'),
                   ("april 31", b'2020-04-31T00:00:00Z'), ("day 00", b'2020-01-00T00:00:00Z'), ("hour 24", b'2020-01-01T24:00:00Z'),
                   ("minute 60", b'2020-01-01T00:60:00Z'), ("second 60", b'2020-01-01T00:00:60Z'), ("lower-case t", b'2020-01-01t00:00:00Z'),
                   ("lower-case z", b'2020-01-01T00:00:00z'), ("no offset", b'2020-01-01T00:00:00'), ("ten fraction digits", b'2020-01-01T00:00:00.1234567890Z'),
                   ("empty fraction", b'2020-01-01T00:00:00.Z'), ("offset hour 24", b'2020-01-01T00:00:00+24:00'), ("offset minute 60", b'2020-01-01T00:00:00+00:60'),
                   ("offset without colon", b'2020-01-01T00:00:00+0000'), ("date only", b'2020-01-01'), ("space separator", b'2020-01-01 00:00:00Z'),
                   ("trailing garbage", b'2020-01-01T00:00:00Zx'), ("empty", b''), ("two-digit year", b'20-01-01T00:00:00Z')]:
    s = b'{"id":1,"shipDate":"' + text + b'"}\n'
    err1("order date: " + name, "order", s, "DATETIME", at(s, b'"shipDate":') + len(b'"shipDate":'))
s = b'{"shipDate":20200101}\n'; err1("order date is a number", "order", s, "TYPE", at(s, b'2020'))
s = b'{"quantity":2147483648}\n'; err1("int32 max + 1", "order", s, "NUM_RANGE", at(s, b'2147'))
s = b'{"quantity":-2147483649}\n'; err1("int32 min - 1", "order", s, "NUM_RANGE", at(s, b'-2147'))
s = b'{"complete":"true"}\n'; err1("bool as a string", "order", s, "TYPE", at(s, b'"true"'))
s = b'{"complete":1}\n'; err1("bool as a number", "order", s, "TYPE", at(s, b':1') + 1)
s = b'{"complete":truE}\n'; err1("bool misspelt", "order", s, "SYNTAX", at(s, b'truE') + 3)
s = b'{"status":"sold"}\n'; err1("Pet literal on an Order", "order", s, "ENUM", at(s, b'"sold"'))
case("order ignores Pet keys", "order", b'{"name":5,"photoUrls":"x","id":3}\n', [{"id": 3}])

# ---- User ------------------------------------------------------------------------------------------
case("user full", "user",
     b'{"id":9,"username":"u1","firstName":"F","lastName":"L","email":"e@x.com","password":"pw","phone":"0123456789","userStatus":3}\n',
     [{"id": 9, "username": "u1", "firstName": "F", "lastName": "L", "email": "e@x.com", "password": "pw", "phone": "0123456789", "userStatus": 3}])
case("user sparse", "user", b'{"phone":"1","userStatus":-1}\n{}\n{"email":null}\n', [{"phone": "1", "userStatus": -1}, {}, {}])
s = b'{"userStatus":3000000000}\n'; err1("userStatus out of int32", "user", s, "NUM_RANGE", at(s, b'3000'))
s = b'{"username":7}\n'; err1("username is a number", "user", s, "TYPE", at(s, b'7'))
s = b'{"firstname":7,"firstName":"x"}\n'; case("user keys are case sensitive", "user", s, [{"firstName": "x"}])

# ---- mixed streams (R12) ---------------------------------------------------------------------------
case("mixed: deciding keys", "mixed",
     b'{"id":1,"name":"a","photoUrls":[]}\n{"id":2,"petId":3}\n{"id":4,"username":"abcdef"}\n{"complete":true}\n{"tags":[],' + MIN + b'}\n',
     [dict(MIN_D, id=1), {"id": 2, "petId": 3}, {"id": 4, "username": "abcdef"}, {"complete": True}, dict(MIN_D, tags=[])])
case("mixed: status before the deciding key", "mixed",
     b'{"status":"sold",' + MIN + b'}\n{"status":"placed","quantity":1}\n{"status":"sold","username":"abcdef"}\n{"id":null,"status":null,"petId":1}\n',
     [dict(MIN_D, status="sold"), {"status": "placed", "quantity": 1}, {"username": "abcdef"}, {"petId": 1}])
s = b'{"id":1}\n'; err1("mixed: only common keys", "mixed", s, "AMBIGUOUS", at(s, b'}'))
s = b'{"id":1,"status":"sold","zzz":[1,2]}\n'; err1("mixed: id + status + unknown", "mixed", s, "AMBIGUOUS", len(s) - 2)
s = b'{}\n'; err1("mixed: empty object", "mixed", s, "AMBIGUOUS", 1)
s = b'{"status":"bogus","petId":1}\n'; err1("mixed: status in neither enum", "mixed", s, "ENUM", at(s, b'"bogus"'))
s = b'{"status":"sold","petId":1}\n'; err1("mixed: Pet literal, then Order key", "mixed", s, "ENUM", at(s, b'"sold"'))
s = b'{"status":"placed",' + MIN + b'}\n'; err1("mixed: Order literal, then Pet key", "mixed", s, "ENUM", at(s, b'"placed"'))
s = b'{"id":"x","petId":1}\n'; err1("mixed: early id of the wrong type", "mixed", s, "TYPE", at(s, b'"x"'))
s = b'{"status":5,"petId":1}\n'; err1("mixed: early status of the wrong type", "mixed", s, "TYPE", at(s, b'5'))
s = b'{"petId":1,"name":"a"}\n'; case("mixed: later keys of another model are unknown", "mixed", s, [{"petId": 1}])
s = b'{"username":"abcdef","status":[1,{"a":2}]}\n'; case("mixed: User has no status", "mixed", s, [{"username": "abcdef"}])
s = b'{"id":1,"name":"a"}\n'; err1("mixed: Pet decided, photoUrls missing", "mixed", s, "REQUIRED", len(s) - 2)
case("mixed: failed records take no row", "mixed", b'{"id":1}\n{"id":2,"petId":3}\n{"petId":"x"}\n{"id":4,"petId":5}\n',
     [("AMBIGUOUS", 7), {"id": 2, "petId": 3}, ("TYPE", 9), {"id": 4, "petId": 5}])

# ---- several records, failures in between --------------------------------------------------------
case("failed records keep an all-absent row", "pet",
     b'{"id":1,' + MIN + b'}\n{"id":x}\n{"id":3,"name":"c","photoUrls":["u"],"tags":[{"id":1}]}\n{"name":"d"}\n',
     [dict(MIN_D, id=1), ("SYNTAX", 6), {"id": 3, "name": "c", "photoUrls": ["u"], "tags": [{"id": 1}]}, ("REQUIRED", 11)])

# ---- array framing -----------------------------------------------------------------------------
A = "array"
case("array: empty", "pet", b'[]', [], A)
case("array: blank inside", "pet", b' [ \n ] \n', [], A)
case("array: two records", "pet", b'[{' + MIN + b'},{"id":1,' + MIN + b'}]', [MIN_D, dict(MIN_D, id=1)], A)
case("array: pretty printed", "pet",
     b'[\n  {\n    "id": 1,\n    "name": "a",\n    "photoUrls": [\n      "u,]"\n    ]\n  },\n  {\n    "name": "b\\"],[",\n    "photoUrls": []\n  }\n]\n',
     [{"id": 1, "name": "a", "photoUrls": ["u,]"]}, {"name": 'b"],[', "photoUrls": []}], A)
s = b'[{' + MIN + b'},]'; case("array: trailing comma", "pet", s, [MIN_D, ("SYNTAX", 0)], A)
s = b'[,]'; case("array: only a comma", "pet", s, [("SYNTAX", 0), ("SYNTAX", 0)], A)
s = b'[{' + MIN + b'}, ,{' + MIN + b'}]'; case("array: hole", "pet", s, [MIN_D, ("SYNTAX", 1), MIN_D], A)
s = b'[{' + MIN + b'} {' + MIN + b'}]'; case("array: missing comma", "pet", s, [("SYNTAX", at(s, b'} {') + 2 - 1)], A)
s = b'[{"name":"a\nb","photoUrls":[]}]'; case("array: raw LF inside a string", "pet", s, [("CTRL_CHAR", at(s, b'\n') - 1)], A)
s = b'[1,{' + MIN + b'},"x"]'; case("array: elements of other types", "pet", s, [("TYPE", 0), MIN_D, ("TYPE", 0)], A)
s = b'x[{' + MIN + b'}]'; case("array: garbage before", "pet", s, [MIN_D, {"doc": ("SYNTAX", 0)}], A)
s = b'[{' + MIN + b'}] y'; case("array: garbage after", "pet", s, [MIN_D, {"doc": ("SYNTAX", len(s) - 1)}], A)
s = b'[{' + MIN + b'}][{' + MIN + b'}]'; case("array: two arrays", "pet", s, [MIN_D, MIN_D, {"doc": ("SYNTAX", at(s, b'][') + 1)}], A)
s = b'[{' + MIN + b'},{"name":"a"'; case("array: input ends inside", "pet", s, [MIN_D, ("EOF", len(b'{"name":"a"')), {"doc": ("EOF", len(s))}], A)
s = b'[{' + MIN + b'},'; case("array: input ends after a comma", "pet", s, [MIN_D, {"doc": ("EOF", len(s))}], A)
s = b''; case("array: empty input", "pet", s, [{"doc": ("EOF", 0)}], A)
# commas at depth 1 separate even without an opening bracket, so the tail of the object is an extent
s = b'{' + MIN + b'}'; case("array: not an array", "pet", s, [("TYPE", 0), {"doc": ("SYNTAX", 0)}], A)
case("array: mixed models", "mixed", b'[{"petId":1},{' + MIN + b'},{"username":"abcdef"}]', [{"petId": 1}, MIN_D, {"username": "abcdef"}], A)


# ---- the other answers of the rules that rest on unobserved behaviour (pj_options.flags) ---------------------
# OPTION_CASES = (name, schema, option bits, input bytes, expected); the same inputs under the default rules are
# covered above (they fail with PJ_E_ENUM / PJ_E_BAD_SURROGATE / PJ_E_TYPE).
ENUM_NULL, LONE_REPLACE, COERCE, HEX_LOWER = 1, 2, 4, 8
OPTION_CASES = []


def ocase(name, schema, opts, data, expected):
    OPTION_CASES.append((name, schema, opts, data, expected))


ocase("enum: unknown literal leaves the property absent", "pet", ENUM_NULL, b'{' + MIN + b',"status":"gone"}\n', [MIN_D])
ocase("enum: known literal still read", "pet", ENUM_NULL, b'{' + MIN + b',"status":"sold"}\n', [dict(MIN_D, status="sold")])
ocase("enum: repeated key, the unknown one last", "pet", ENUM_NULL, b'{' + MIN + b',"status":"sold","status":"Sold"}\n', [MIN_D])
ocase("enum: order", "order", ENUM_NULL, b'{"status":"x","quantity":1}\n{"status":"placed"}\n', [{"quantity": 1}, {"status": "placed"}])
ocase("enum: mixed stream, status before the deciding key", "mixed", ENUM_NULL,
      b'{"id":1,"status":"zzz","petId":2}\n{"status":"sold","petId":2}\n{"status":"sold","name":"a","photoUrls":[]}\n',
      [{"id": 1, "petId": 2}, {"petId": 2}, dict(MIN_D, status="sold")])
ocase("enum: other failures stay failures", "pet", ENUM_NULL, b'{' + MIN + b',"status":5}\n{"status":"gone"}\n',
      [("TYPE", at(b'{' + MIN + b',"status":5}', b'5')), ("REQUIRED", len(b'{"status":"gone"') )])

ocase("surrogate: lone high and lone low become U+FFFD", "pet", LONE_REPLACE,
      b'{"name":"\\ud800","photoUrls":["\\udc00x","\\ud83d\\u0041","\\ud83d\\ud83d\\ude00","a\\udfffb"]}\n',
      [{"name": "�", "photoUrls": ["�x", "�A", "�\U0001F600", "a�b"]}])
ocase("surrogate: pairs still pair", "pet", LONE_REPLACE, b'{"name":"\\ud83d\\ude00","photoUrls":[]}\n', [{"name": "\U0001F600", "photoUrls": []}])
ocase("surrogate: a bad escape after a lone high is still a bad escape", "pet", LONE_REPLACE, b'{"name":"\\ud800\\u12","photoUrls":[]}\n',
      [("BAD_ESCAPE", at(b'{"name":"\\ud800\\u12"', b'"', 3))])

ocase("coerce: integers from strings, strings from numbers and booleans", "pet", COERCE,
      b'{"id":"12","category":{"id":"-3","name":true},"name":5,"photoUrls":[]}\n{"name":-1.5e3,"photoUrls":[],"tags":[{"id":"0","name":0}]}\n',
      [{"id": 12, "category": {"id": -3, "name": "true"}, "name": "5", "photoUrls": []},
       {"name": "-1.5e3", "photoUrls": [], "tags": [{"id": 0, "name": "0"}]}])
ocase("coerce: a string that is no integer", "pet", COERCE, b'{"id":"1.0",' + MIN + b'}\n{"id":"",' + MIN + b'}\n{"id":"01",' + MIN + b'}\n{"id":" 1",' + MIN + b'}\n',
      [("TYPE", 6), ("TYPE", 6), ("TYPE", 6), ("TYPE", 6)])
ocase("coerce: range of the integer in the string", "pet", COERCE,
      b'{"id":"9223372036854775807",' + MIN + b'}\n{"id":"9223372036854775808",' + MIN + b'}\n{"id":"-9223372036854775808",' + MIN + b'}\n',
      [dict(MIN_D, id=9223372036854775807), ("NUM_RANGE", 6), dict(MIN_D, id=-9223372036854775808)])
ocase("coerce: order", "order", COERCE, b'{"complete":"true","quantity":"7","petId":"8"}\n{"complete":"yes"}\n{"quantity":"2147483648"}\n',
      [{"petId": 8, "quantity": 7, "complete": True}, ("TYPE", 12), ("NUM_RANGE", 12)])
ocase("coerce: user", "user", COERCE, b'{"phone":5551234,"userStatus":"2","email":false}\n', [{"email": "false", "phone": "5551234", "userStatus": 2}])
ocase("coerce: mixed stream, id before the deciding key", "mixed", COERCE, b'{"id":"7","username":1}\n', [{"id": 7, "username": "1"}])
ocase("coerce: list elements, enums and date-times are not coerced", "pet", COERCE,
      b'{"name":"a","photoUrls":[1]}\n{' + MIN + b',"status":1}\n{"name":[],"photoUrls":[]}\n',
      [("TYPE", at(b'{"name":"a","photoUrls":[1', b'1')), ("TYPE", at(b'{' + MIN + b',"status":1', b'1')), ("TYPE", at(b'{"name":[', b'['))])
ocase("coerce: a malformed number is still a syntax failure", "pet", COERCE, b'{"name":01,"photoUrls":[]}\n', [("SYNTAX", at(b'{"name":01', b'1'))])
