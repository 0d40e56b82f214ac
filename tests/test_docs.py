"""The pages under docs/ stay in step with the code: every environment variable the sources read is documented, every
documented algorithm name is registered, and every C function the pages mention is exported by the library."""
import ctypes
import pathlib
import re

from hccl_b200._lib import lib

ROOT = pathlib.Path(__file__).resolve().parents[1]
DOCS = ROOT / "docs"


def _sources():
    for sub, pats in (("csrc", ("*.cc", "*.cu", "*.cuh", "*.h")), ("hccl_b200", ("*.py",))):
        for pat in pats:
            yield from (ROOT / sub).rglob(pat)


def test_every_environment_variable_read_by_the_sources_is_documented():
    text = (DOCS / "env_variables.md").read_text()
    documented = set(re.findall(r"`(HCCL_[A-Z0-9_]+)`", text))
    read = set()
    for path in _sources():
        read |= set(re.findall(r"getenv\(\"(HCCL_[A-Z0-9_]+)\"\)", path.read_text(errors="ignore")))
        read |= set(re.findall(r"environ(?:\.get)?[\[(]\"(HCCL_[A-Z0-9_]+)\"", path.read_text(errors="ignore")))
    # variables parsed through the table in env_config.cc
    read |= set(re.findall(r"\{\"(HCCL_[A-Z0-9_]+)\", Parse", (ROOT / "csrc/common/env_config.cc").read_text()))
    read |= set(re.findall(r"(?:flag|u32)\(\"(HCCL_[A-Z0-9_]+)\"", (ROOT / "csrc/common/env_config.cc").read_text()))
    assert len(read) > 40
    assert read - documented == set(), sorted(read - documented)


def test_documented_algorithm_names_are_the_registered_ones():
    l = lib()
    registered = set()
    for op in range(1, 37):
        buf = ctypes.create_string_buffer(1 << 14)
        if l.HcclListAlgorithms(op, buf, 1 << 14) == 0:
            registered |= {n for n in buf.value.decode().split(";") if n}
    text = (DOCS / "algorithms.md").read_text()
    table = "\n".join(ln for ln in text.splitlines() if ln.startswith("| "))
    documented = set(re.findall(r"`((?:Nvls|Sm|Ins|Reduce)[A-Za-z0-9]+)`", table))
    assert len(registered) > 60
    assert documented == registered, (sorted(documented - registered), sorted(registered - documented))


def test_c_functions_named_in_the_docs_are_exported():
    l = lib()
    names = set()
    for page in DOCS.glob("*.md"):
        names |= set(re.findall(r"`(Hccl[A-Z][A-Za-z0-9]+)(?:\(|`)", page.read_text()))
    names -= {"HcclResult", "HcclComm", "HcclCommConfig", "HcclRootInfo", "HcclCMDType", "HcclSendRecvItem"}
    assert len(names) > 40
    missing = [n for n in sorted(names) if not hasattr(l, n)]
    assert missing == [], missing


def test_api_index_lists_exactly_the_functions_the_headers_declare():
    l = lib()
    index = (DOCS / "api_index.md").read_text()
    sections = dict(re.findall(r"## `(hccl[a-z_0-9]*\.h)`\n(.*?)(?=\n## |\Z)", index, flags=re.S))
    for header in sorted((ROOT / "include" / "hccl").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        declared = set(re.findall(r"\b(Hccl[A-Z][A-Za-z0-9]+)\s*\(", text))
        listed = set(re.findall(r"`(Hccl[A-Z][A-Za-z0-9]+)`", sections.get(header.name, ""))) - {"HcclCommConfig", "HcclRootInfo", "HcclSendRecvItem"}
        assert header.name in sections, header.name
        assert declared == listed - ({"HcclMemAlloc"} if header.name != "hccl_res.h" else set()), (header.name, sorted(declared ^ listed))
        for name in declared:
            assert hasattr(l, name), name                       # and the library exports every one of them


def test_testing_page_names_every_test_file_and_only_existing_ones():
    text = (DOCS / "testing.md").read_text()
    cited = set(re.findall(r"`(test_[a-z0-9_]+\.py)`", text))
    existing = {p.name for p in (ROOT / "tests").glob("test_*.py")}
    assert cited == existing, (sorted(cited - existing), sorted(existing - cited))
