"""Source-level guarantees that need no GPU: no cluster-multicast bulk loads, no unbounded traps,
SM-budget model behaviour, packaging of native sources."""

import math
import re
from pathlib import Path

from nanoep_b200.utils import sms
from nanoep_b200.utils.build import SOURCES, source_dir

ROOT = Path(__file__).resolve().parent.parent


def _native_sources():
    return [p for p in (ROOT / "csrc").rglob("*") if p.suffix in {".cu", ".cuh", ".hpp", ".cpp", ".h"}]


def test_no_cluster_multicast_loads_and_no_traps():
    # patterns are assembled from pieces so that this file does not itself contain them
    banned = re.compile("|".join(["multi" + "cast::cluster", "_MULTI" + "CAST", r"__tr" + r"ap\s*\(", r"asm[^;]*\btr" + r"ap;", "Memcpy" + "Batch" + "Async"]))
    for path in _native_sources():
        text = path.read_text()
        assert not banned.search(text), f"{path} uses a construct that is banned in this project"


def _loops(text):
    """(header, body) of every `for`/`while`/`do` loop in C-like source; bodies are brace-matched, a loop
    without braces ends at its first semicolon."""
    for m in re.finditer(r"\b(for|while|do)\b", text):
        i = m.end()
        header = ""
        if m.group(1) != "do":
            while i < len(text) and text[i].isspace():
                i += 1
            if i >= len(text) or text[i] != "(":
                continue
            depth, j = 0, i
            while j < len(text):
                depth += text[j] == "("
                depth -= text[j] == ")"
                j += 1
                if depth == 0:
                    break
            header, i = text[i:j], j
        while i < len(text) and text[i].isspace():
            i += 1
        if i < len(text) and text[i] == "{":
            depth, j = 0, i
            while j < len(text):
                depth += text[j] == "{"
                depth -= text[j] == "}"
                j += 1
                if depth == 0:
                    break
            body = text[i:j]
        else:
            j = text.find(";", i)
            body = text[i : j + 1]
            if m.group(1) == "while" and not body.strip(" ;"):
                continue  # the tail of a do { } while (...);
        yield header, body


def test_every_device_wait_is_bounded():
    """Every loop in the native sources that polls memory, an mbarrier or sleeps must compare a timer (or an
    iteration count) against a limit inside the loop."""
    polls = re.compile(r"ld_acquire|ld_relaxed_sys|try_wait|mbar_try|__nanosleep|volatile")
    bounded = re.compile(r"timeout_ns|limit_ns|deadline|max_spins|kMaxSpins")
    # a counted loop (declares its index, compares it with a bound, steps it) ends by itself unless its header polls
    counted = re.compile(r"^\(\s*(?:int|unsigned|int64_t|uint32_t|size_t)\s+\w+\s*=[^;]*;[^;]*[<>][^;]*;[^;]*(?:\+=|\+\+|-=|--)[^;]*\)$", re.S)
    checked = 0
    for path in _native_sources():
        if path.suffix == ".cpp" or path.name.endswith(".hpp"):
            continue  # host code: its waits are wall-clock bounded and tested separately
        text = re.sub(r"//[^\n]*", "", path.read_text())
        for header, body in _loops(text):
            if counted.match(header.strip()) and not polls.search(header):
                continue
            if polls.search(header) or (polls.search(body) and re.search(r"\b(break|return)\b", body) and not re.search(r"\bfor\b|\bwhile\b", body[1:])):
                checked += 1
                assert bounded.search(header + body), f"{path.name}: unbounded wait loop: {header} {body[:200]}"
    assert checked >= 6, "the scan found no wait loops; the patterns are stale"


def test_build_lists_existing_sources():
    for name in SOURCES:
        assert (source_dir() / name).exists(), name


def test_sm_budget_model():
    assert sms.theoretical_num_sms(148, 1, 256, 8, 810.0) == 148
    assert sms.theoretical_num_sms(148, 8, 256, 8, 0.0) == 148  # unknown NVLink -> all SMs
    n = sms.theoretical_num_sms(148, 8, 256, 8, 810.0)
    assert 16 <= n <= 148 and n % 4 == 0
    assert sms.theoretical_num_sms(148, 2, 64, 6, 810.0) <= 148
    p = sms.send_probability(8, 256, 8)
    assert abs(p - (1 - math.comb(224, 8) / math.comb(256, 8))) < 1e-12
    assert sms.nvlink_gbs(("a",)) == 0.0
    assert sms.nvlink_gbs(("no-such-gpu-1", "no-such-gpu-2")) == 0.0  # nvidia-smi missing or GPUs unknown


def test_nvtx_range_is_a_shared_noop_when_disabled():
    from nanoep_b200.utils import tracing

    if not tracing._ENABLED:
        assert tracing.nvtx_range("a") is tracing.nvtx_range("b")
    with tracing.nvtx_range("anything"):
        pass
