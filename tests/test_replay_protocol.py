"""The replay program's side of its protocol, with a stand-in engine: one JSON object a line in, a
`done <step>` line after every step, `<step>.f32` only for steps in which something is wanted, rows
in the order of the entries and of `want`, requests ended when the step says so. No GPU needed; the
real engine behind the same program is tested with `-m gpu`."""
import io
import json

import numpy as np
import torch

import kapel_b200.engine.replay as replay
import kapel_b200.engine.step as step_module

VOCAB = 7


class StandInEngine:
    """Logits that name their request's position: row[j] = 1000 * (hash of id) + position + j / 10."""

    made = []

    def __init__(self):
        self.lengths, self.ended, self.steps = {}, [], []

    @classmethod
    def from_dir(cls, folder, dtype, max_tokens, max_sequences):
        eng = cls()
        eng.args = (str(folder), dtype, max_tokens, max_sequences)
        cls.made.append(eng)
        return eng

    def step(self, entries):
        rows = []
        self.steps.append([(e.id, list(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            start = self.lengths.get(e.id, 0)
            for w in e.want:
                rows.append([1000.0 * (sum(map(ord, str(e.id))) % 50) + start + w + j / 10 for j in range(VOCAB)])
            self.lengths[e.id] = start + len(e.tokens)
        return torch.tensor(rows, dtype=torch.float32).reshape(-1, VOCAB)

    def end(self, seq_id):
        self.ended.append(seq_id)
        self.lengths.pop(seq_id, None)


def test_steps_in_done_lines_and_files_out(monkeypatch, tmp_path, capsys):
    monkeypatch.setattr(step_module, "Engine", StandInEngine)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [9], "want": []}, {"id": "b", "tokens": [1, 2], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": [4, 4, 4], "want": [2, 0]}, {"id": "a", "tokens": [8], "want": [0]}], "end": ["a"]},
        {"step": 7, "entries": [], "end": ["b"]},
    ]
    monkeypatch.setattr("sys.stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n\n"))
    out = tmp_path / "logits"
    assert replay.main(["--model", "DIR", "--dtype", "float32", "--out", str(out), "--max-tokens", "128"]) == 0
    printed = capsys.readouterr()
    assert printed.out.split("\n")[:4] == ["done 0", "done 1", "done 2", "done 7"]       # nothing else on standard output
    eng = StandInEngine.made[-1]
    assert eng.args == ("DIR", "float32", 128, 16)
    assert eng.ended == ["a", "b"]
    assert sorted(p.name for p in out.iterdir()) == ["0.f32", "2.f32"]                   # steps 1 and 7 want nothing
    first = np.frombuffer((out / "0.f32").read_bytes(), dtype="<f4").reshape(-1, VOCAB)
    assert first.shape == (2, VOCAB) and first[0, 0] == first[1, 0] - 2                   # places 0 and 2 of a's prompt
    third = np.frombuffer((out / "2.f32").read_bytes(), dtype="<f4").reshape(-1, VOCAB)
    hb, ha = 1000.0 * (ord("b") % 50), 1000.0 * (ord("a") % 50)
    assert third[:, 0].tolist() == [hb + 2 + 2, hb + 2 + 0, ha + 4 + 0]                   # b's rows in the order of `want`, then a's
    assert eng.steps[1] == [("a", [9], []), ("b", [1, 2], [])]


def test_max_tokens_must_be_positive(monkeypatch, tmp_path):
    monkeypatch.setattr(step_module, "Engine", StandInEngine)
    try:
        replay.main(["--model", "DIR", "--dtype", "bfloat16", "--out", str(tmp_path), "--max-tokens", "0"])
    except SystemExit as err:
        assert err.code == 2
    else:
        raise AssertionError("a pool of no tokens was accepted")
