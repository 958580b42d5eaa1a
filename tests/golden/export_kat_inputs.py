"""Writes the known-answer inputs (tests/golden/kat_cases.py) as JSON lines for tests/golden/EmitGolden.java:

    python tests/golden/export_kat_inputs.py > kat_inputs.jsonl

Each line: {"name", "schema", "framing", "input_b64"}. The Java program answers with java_golden.jsonl, which
tests/test_oracle_kat.py picks up when it lies beside this file.
"""
import base64
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from golden.kat_cases import CASES  # noqa: E402


def lines():
    for name, schema, framing, data, _expected in CASES:
        yield json.dumps({"name": name, "schema": schema, "framing": framing, "input_b64": base64.b64encode(bytes(data)).decode()})


if __name__ == "__main__":
    for ln in lines():
        print(ln)
