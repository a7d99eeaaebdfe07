"""The replay program's protocol with a stand-in for the model runner (CPU): which calls a trace turns
into, the files it writes and the lines it prints.  The numbers themselves are the GPU tests' business."""

import io
import json

import numpy as np
import torch

from prism_b200.engine import replay

V = 7


class FakeRunner:
    def __init__(self):
        self.calls, self.lengths = [], {}

    def begin_request(self, rid):
        assert rid not in self.lengths
        self.lengths[rid] = 0
        self.calls.append(("begin", rid))

    def end_request(self, rid):
        del self.lengths[rid]
        self.calls.append(("end", rid))

    def check_errors(self):
        self.calls.append(("check",))

    def step(self, segs):
        self.calls.append(("step", [(s.req_id, list(s.tokens), list(s.want)) for s in segs]))
        rows = []
        for s in segs:
            for w in s.want:
                # a row that names its request's position and token
                rows.append(torch.full((V,), float(100 * (self.lengths[s.req_id] + w) + s.tokens[w])))
            self.lengths[s.req_id] += len(s.tokens)
        return torch.stack(rows) if rows else None


def run(monkeypatch, tmp_path, capsys, lines, extra=()):
    fake = FakeRunner()
    seen = {}

    def build_runner(model_dir, dtype, max_tokens, page_size, max_live, device="cuda:0"):
        seen.update(model=model_dir, dtype=dtype, max_tokens=max_tokens, page_size=page_size)
        return None, None, None, fake
    monkeypatch.setattr(replay, "build_runner", build_runner)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "set_device", lambda d: None)
    monkeypatch.setattr("sys.stdin", io.StringIO("".join(json.dumps(x) + "\n" if not isinstance(x, str) else x for x in lines)))
    out = tmp_path / "out"
    rc = replay.main(["--model", "M", "--dtype", "float32", "--out", str(out), "--max-tokens", "128", *extra])
    return rc, fake, seen, out, capsys.readouterr().out


def test_steps_files_and_done_lines(monkeypatch, tmp_path, capsys):
    lines = [
        {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []},
        "\n",                                                                     # an empty line is skipped
        {"step": 1, "entries": [{"id": "a", "tokens": [7], "want": [0]},
                                {"id": "b", "tokens": [1, 2], "want": []}], "end": ["a"]},
        {"step": 2, "entries": [{"id": "b", "tokens": [4, 4], "want": [1, 0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": [9, 9], "want": []}], "end": []},      # the id may come again
    ]
    rc, fake, seen, out, printed = run(monkeypatch, tmp_path, capsys, lines)
    assert rc == 0 and seen == dict(model="M", dtype="float32", max_tokens=128, page_size=64)
    assert printed.split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    # logits files: only for steps in which something was wanted; order of the entries and of `want`
    assert sorted(p.name for p in out.iterdir()) == ["0.f32", "1.f32", "2.f32"]
    f0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)
    f1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V)
    f2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V)
    assert f0[:, 0].tolist() == [5.0, 203.0] and f1[:, 0].tolist() == [307.0]
    assert f2[:, 0].tolist() == [304.0, 204.0]                                   # want [1, 0]: that order
    # the calls: a request begins at its first entry, ends after the step that names it in `end`
    kinds = [c[0] for c in fake.calls]
    assert kinds == ["begin", "step", "check", "begin", "step", "end", "check", "step", "end", "check",
                     "begin", "step", "check"]
    assert fake.calls[4][1] == [("a", [7], [0]), ("b", [1, 2], [])]              # one batch, in the trace's order
    assert fake.lengths == {"a": 2}                                              # the second "a" started from nothing


def test_an_entry_without_tokens_is_left_out_of_the_batch(monkeypatch, tmp_path, capsys):
    lines = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2], "want": [1]}, {"id": "b", "tokens": [], "want": []}],
              "end": ["b"]}]
    rc, fake, _, out, printed = run(monkeypatch, tmp_path, capsys, lines, extra=["--page-size", "16"])
    assert rc == 0 and printed.strip() == "done 0"
    assert [c for c in fake.calls if c[0] == "step"][0][1] == [("a", [1, 2], [1])]
    assert ("begin", "b") in fake.calls and ("end", "b") in fake.calls


def test_no_gpu_is_an_error_not_a_fallback(monkeypatch, tmp_path, capsys):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    monkeypatch.setattr("sys.stdin", io.StringIO(""))
    assert replay.main(["--model", "M", "--out", str(tmp_path / "o"), "--max-tokens", "64"]) == 1
