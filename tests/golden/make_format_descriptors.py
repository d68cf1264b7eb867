"""Writes tests/golden/reference_format_descriptors.json from the reference's own source.

Parses the `self.insert(QuantFormatDescriptor { ... })` literals of gllm-kernels' src/quant_format.rs (the
registry behind QuantFormatDescriptor::for_type) and records, for the nine formats this library serves, every
field as the reference wrote it: enum variants by name, their payload fields as integers.  Nothing is computed by
this project's code.  Needs the reference checkout; the JSON it writes is what travels.

Run:  python tests/golden/make_format_descriptors.py path/to/gllm-kernels
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
WANT = ["Q4_0", "Q5_0", "Q8_0", "Q4_K", "Q5_K", "Q6_K", "Q8_K", "MXFP4", "NVFP4"]


def strip_comments(text: str) -> str:
    return re.sub(r"//[^\n]*", "", text)


def split_top_level(body: str):
    """`a: X, b: Y { c: 1, d: 2 }, ...` -> [(a, X), (b, 'Y { c: 1, d: 2 }'), ...] (commas inside braces kept)."""
    out, depth, cur = [], 0, ""
    for ch in body:
        if ch in "{(":
            depth += 1
        elif ch in "})":
            depth -= 1
        if ch == "," and depth == 0:
            if cur.strip():
                out.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur.strip())
    return [tuple(s.strip() for s in item.split(":", 1)) for item in out]


def parse_value(v: str):
    v = v.strip()
    m = re.match(r"^(?:Some\()?([A-Za-z_:0-9]+)\s*\{(.*)\}\)?$", v, re.S)
    if m:  # enum variant with named fields
        fields = {k: parse_value(x) for k, x in split_top_level(m.group(2))}
        return {"variant": m.group(1).split("::")[-1], **fields}
    m = re.match(r"^Some\((.*)\)$", v, re.S)
    if m:
        return parse_value(m.group(1))
    if v == "None":
        return None
    if re.match(r"^-?\d+$", v):
        return int(v)
    if v in ("true", "false"):
        return v == "true"
    if v.startswith('"'):
        return v.strip('"')
    return v.split("::")[-1]  # bare enum variant


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_format_descriptors.py <checkout of gllm-kernels>")
    ref = sys.argv[1]
    path = os.path.join(ref, "src", "quant_format.rs")
    raw = open(path).read()
    text = strip_comments(raw)
    out = {"cite": "src/quant_format.rs (QuantFormatRegistry::register_classic / register_kquant / register_external)", "formats": {}}
    for m in re.finditer(r"self\.insert\(QuantFormatDescriptor\s*\{", text):
        i, depth = m.end(), 1
        while depth:
            depth += {"{": 1, "}": -1}.get(text[i], 0)
            i += 1
        fields = {k: parse_value(v) for k, v in split_top_level(text[m.end():i - 1])}
        if fields.get("name") in WANT:
            fields["line"] = raw[:raw.index(f'name: "{fields["name"]}"')].count("\n") + 1
            out["formats"][fields["name"]] = fields
    missing = [n for n in WANT if n not in out["formats"]]
    assert not missing, missing
    with open(os.path.join(HERE, "reference_format_descriptors.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote", len(out["formats"]), "descriptors")


if __name__ == "__main__":
    main()
