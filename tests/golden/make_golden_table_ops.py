"""Generate ``table_ops.npz``: what the reference's own batch / page-table helpers return on seeded inputs.

    python tests/golden/make_golden_table_ops.py --reference <easymlx checkout>

The helpers live on ``ModelRunner`` (inference/esurge/runners/model_runner.py) and ``BaseCausalLMModule``
(modules/_base/causal_lm_module.py); importing those modules pulls in the whole engine, so the script takes the
method definitions out of the files with ``ast`` at run time, compiles them unchanged against the NumPy stand-in
for ``mlx.core`` (``mlx_shim/``) and calls them on a bare object that carries only the attributes they touch.
Nothing of the reference is stored in this repository: only the inputs' seeds and the returned arrays.
"""

from __future__ import annotations

import __future__
import argparse
import ast
import os
import sys
import types
from collections import namedtuple

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

SCHEDULER_METHODS = ("_make_prefill_slice", "_make_decode_slice")
RUNNER_METHODS = ("_build_positions", "_clear_row_mapping", "_page_ids_array", "_copy_cache_row", "_zero_indexed_cache_rows", "_zero_pages",
                  "_assign_row_mapping", "_move_cache_row", "compact_rows", "_flatten_sequence_tokens",
                  "_get_compiled_batch_padder", "_pad_batch_token_ids")
MODULE_METHODS = ("_extract_last_tokens",)


def extract_methods(path: str, class_names: tuple[str, ...], wanted: tuple[str, ...], env: dict) -> dict:
    tree = ast.parse(open(path).read())
    found = {}
    for node in tree.body:
        if isinstance(node, ast.ClassDef) and node.name in class_names:
            for item in node.body:
                if isinstance(item, ast.FunctionDef) and item.name in wanted:
                    static = any(isinstance(d, ast.Name) and d.id == "staticmethod" for d in item.decorator_list)
                    item.decorator_list = []
                    module = ast.Module(body=[item], type_ignores=[])
                    code = compile(module, path, "exec", flags=__future__.annotations.compiler_flag)
                    scope = dict(env)
                    exec(code, scope)
                    fn = scope[item.name]
                    found[item.name] = staticmethod(fn) if static else fn
    missing = set(wanted) - set(found)
    if missing:
        raise SystemExit(f"{path}: methods not found: {sorted(missing)}")
    return found


class _Buffer:
    def __init__(self, moves):
        self._moves = moves

    def compact_holes(self):
        return list(self._moves)

    def trim_trailing_holes(self):
        return None


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.join(HERE, "table_ops.npz"))
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(HERE, "mlx_shim"))
    import mlx.core as mx

    root = os.path.join(args.reference, "lib", "python", "easymlx")
    Seq = namedtuple("ScheduledSequence", "token_ids")
    env = {"mx": mx, "Any": object, "_safe_eval": lambda *a, **k: None, "ScheduledSequence": Seq}
    runner_cls = type("Runner", (), extract_methods(os.path.join(root, "inference", "esurge", "runners", "model_runner.py"),
                                                    ("ModelRunner",), RUNNER_METHODS, env))
    lm_cls = type("LM", (), extract_methods(os.path.join(root, "modules", "_base", "causal_lm_module.py"),
                                            ("BaseCausalLMModule",), MODULE_METHODS, {"mx": mx, "PageMetadata": object}))
    out: dict[str, np.ndarray] = {}
    rng = np.random.default_rng(77)

    # ---- page-table rows
    slots, mb, nb, bs, hkv, d = 6, 5, 12, 4, 2, 8
    bt0 = rng.integers(-1, nb, size=(slots, mb)).astype(np.int32)
    lens0 = rng.integers(0, mb * bs, size=slots).astype(np.int32)
    k0 = rng.standard_normal((nb, bs, hkv, d)).astype(np.float16)
    v0 = rng.standard_normal((nb, bs, hkv, d)).astype(np.float16)
    out.update(bt0=bt0, lens0=lens0, k0=k0, v0=v0)

    def runner(moves=()):
        r = runner_cls()
        cache = types.SimpleNamespace(block_tables=mx.array(bt0.copy()), kv_lens=mx.array(lens0.copy()),
                                      key_cache=mx.array(k0.copy()), value_cache=mx.array(v0.copy()))
        r.kv_caches = [cache]
        r.sequence_buffer = _Buffer(moves)
        r._compiled_batch_padders = {}
        return r, cache

    r, c = runner()
    r._assign_row_mapping(2, [7, 3, 9], cached_tokens=5)
    r._assign_row_mapping(4, [1, 2, 3, 4, 5, 6, 7], cached_tokens=-3)
    out.update(assign_bt=np.asarray(c.block_tables), assign_lens=np.asarray(c.kv_lens))
    r, c = runner()
    r._move_cache_row(1, 4)
    r._move_cache_row(3, 3)
    out.update(swap_bt=np.asarray(c.block_tables), swap_lens=np.asarray(c.kv_lens))
    moves = [(3, 0), (5, 1), (4, 3)]
    r, c = runner(moves)
    got = r.compact_rows()
    assert [tuple(m) for m in got] == moves
    out.update(compact_moves=np.asarray(moves, dtype=np.int32), compact_bt=np.asarray(c.block_tables),
               compact_lens=np.asarray(c.kv_lens))
    r, c = runner()
    r._clear_row_mapping(2)
    out.update(clear_bt=np.asarray(c.block_tables), clear_lens=np.asarray(c.kv_lens))
    r, c = runner()
    zero_ids = [3, -1, 11, 40, 3]
    r._zero_pages(zero_ids)
    out.update(zero_ids=np.asarray(zero_ids, dtype=np.int32), zero_k=np.asarray(c.key_cache), zero_v=np.asarray(c.value_cache))

    # ---- packed ids
    token_lists = [[5, 6, 7], [11], [], [21, 22, 23, 24, 25], [31, 32]]
    r, _ = runner()
    flat, qlens = r._flatten_sequence_tokens([Seq(t) for t in token_lists])
    padded, qlens2 = r._pad_batch_token_ids([Seq(t) for t in token_lists])
    assert qlens == qlens2
    out.update(ids_flat=np.asarray(flat), ids_lens=np.asarray(qlens, dtype=np.int32), ids_padded=np.asarray(padded))

    # ---- last tokens
    hidden = rng.standard_normal((int(np.sum(qlens)), 16)).astype(np.float32)
    qsl = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    meta = types.SimpleNamespace(query_start_loc=mx.array(qsl), is_single_token_decode=False)
    last = lm_cls()._extract_last_tokens(mx.array(hidden), meta)
    out.update(last_hidden=hidden, last_qsl=qsl, last_out=np.asarray(last))

    # ---- scheduler slices and positions (scheduler/scheduler.py:327-372, model_runner.py:1292-1306)
    sched_cls = type("Sched", (), extract_methods(os.path.join(root, "inference", "esurge", "scheduler", "scheduler.py"),
                                                  ("Scheduler",), SCHEDULER_METHODS, {"EngineRequest": object}))
    cases = []
    prompt = list(range(100, 140))
    for computed, budget, chunked, threshold in [(0, 64, False, None), (0, 16, False, None), (8, 64, True, 12),
                                                 (35, 64, True, 12), (40, 64, True, 12), (3, 0, True, 12), (3, 7, True, 0)]:
        sch = sched_cls()
        sch.scheduler_config = types.SimpleNamespace(long_prefill_token_threshold=threshold, chunked_prefill_enabled=chunked)
        req = types.SimpleNamespace(remaining_prefill_tokens=len(prompt) - computed, num_computed_tokens=computed,
                                    all_token_ids=prompt)
        ids, count = sch._make_prefill_slice(req, budget)
        cases.append([computed, budget, int(chunked), -1 if threshold is None else threshold, count] + list(ids) + [-1] * (64 - len(ids)))
    out["prefill_slices"] = np.asarray(cases, dtype=np.int32)
    dcases = []
    for generated, prm, gen_budget, budget in [([7, 8, 9], [1, 2], 5, 3), ([], [1, 2], 5, 3), ([], [], 5, 3), ([4], [1], 0, 3), ([4], [1], 2, 0)]:
        sch = sched_cls()
        req = types.SimpleNamespace(generated_token_ids=generated, prompt_token_ids=prm, remaining_generation_budget=gen_budget)
        ids, count = sch._make_decode_slice(req, budget)
        dcases.append([len(generated), len(prm), gen_budget, budget, count, ids[0] if ids else -1])
    out["decode_slices"] = np.asarray(dcases, dtype=np.int32)
    SeqP = namedtuple("SeqP", "token_ids num_computed_tokens")
    pos = runner_cls._build_positions([SeqP([1, 2, 3], 5), SeqP([9], 0), SeqP([], 4), SeqP([1, 1], 127)])
    out["positions_flat"] = np.asarray([p for row in pos for p in row], dtype=np.int32)

    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {sorted(out)}")


if __name__ == "__main__":
    main()
