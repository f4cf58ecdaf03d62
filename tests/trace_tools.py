"""Building traces for bin/trace_run and reading what it writes."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def whole_trace(requests):
    """Each request alone and whole: one step per request, logits everywhere."""
    steps, index = [], []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
        index.append([(rid, p) for p in range(len(toks))])
    return steps, index


def tail_trace(requests, tail=32):
    """The first n - tail tokens in one step, then the last ``tail`` one by one."""
    steps, index, k = [], [], 0
    for rid, toks in requests.items():
        n = len(toks)
        head = max(1, n - tail)
        steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": [rid] if head == n else []})
        index.append([(rid, p) for p in range(head)])
        k += 1
        for p in range(head, n):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == n - 1 else []})
            index.append([(rid, p)])
            k += 1
    return steps, index


def batched_trace(requests, batch_size, prompt_frac=0.5):
    """Batches that start together: the first step brings a prefix of each request, later steps one
    token each; shorter requests end earlier; one batch after another."""
    steps, index, k = [], [], 0
    rids = list(requests)
    for b0 in range(0, len(rids), batch_size):
        group = rids[b0:b0 + batch_size]
        fed = {}
        entries, idx, end = [], [], []
        for rid in group:
            toks = requests[rid]
            head = max(1, int(len(toks) * prompt_frac))
            entries.append({"id": rid, "tokens": toks[:head], "want": list(range(head))})
            idx.extend((rid, p) for p in range(head))
            fed[rid] = head
            if head == len(toks):
                end.append(rid)
        steps.append({"step": k, "entries": entries, "end": end})
        index.append(idx)
        k += 1
        live = [r for r in group if fed[r] < len(requests[r])]
        while live:
            entries, idx, end = [], [], []
            for rid in live:
                p = fed[rid]
                entries.append({"id": rid, "tokens": [requests[rid][p]], "want": [0]})
                idx.append((rid, p))
                fed[rid] = p + 1
                if fed[rid] == len(requests[rid]):
                    end.append(rid)
            steps.append({"step": k, "entries": entries, "end": end})
            index.append(idx)
            k += 1
            live = [r for r in live if fed[r] < len(requests[r])]
    return steps, index


def run_trace(model_dir, dtype, steps, out_dir, max_tokens, env=None):
    """Feed ``steps`` to bin/trace_run; returns {step: float32 array [wanted, vocab]}."""
    os.makedirs(out_dir, exist_ok=True)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
                        "--max-tokens", str(max_tokens)], input=text, capture_output=True, text=True, env=env)
    assert p.returncode == 0, p.stderr[-4000:]
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], p.stdout[-2000:]
    return p


def collect(out_dir, steps, index, vocab):
    """{(request id, position): logits row} from the files of a replay."""
    rows = {}
    for s, idx in zip(steps, index):
        n_want = sum(len(e["want"]) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if n_want == 0:
            assert not os.path.exists(path)
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(n_want, vocab)
        for key, row in zip(idx, arr):
            rows[key] = row
    return rows
