"""Turn raw RL datasets into the local files the data loaders read (``unirl_b200/data/datasets.py``).

``dapo-math``   competition math for rule-verified rewards: ``train.jsonl`` from a DAPO-Math-17k style table and ``aime_eval.jsonl``
                from one or more AIME style tables, one ``{"prompt", "metadata": {"answer"}}`` record per problem.
``geo3k-mc``    multiple-choice geometry with a diagram: ``{train,val,test}.jsonl`` with the choices written into the prompt, the letter of
                the right choice in ``metadata.answer`` and the diagram saved under ``images/`` and referenced through ``media_refs``
                (relative to the jsonl's folder).

A source is a local ``.parquet`` / ``.jsonl`` file, or — when the ``datasets`` package is installed and the machine is online — a hub
id written as ``hub:<id>[:<split>]``.  Column names vary between sources; the extractors accept the usual ones (chat-style ``prompt``
lists with ``reward_model.ground_truth``, plain ``problem`` / ``question`` + ``answer`` / ``solution`` columns, capitalised variants).

    python -m unirl_b200.tools.prepare_data dapo-math --train dapo.parquet --eval aime24.parquet aime25.parquet --out-dir data/dapo_math
    python -m unirl_b200.tools.prepare_data geo3k-mc --train geo_train.parquet --val geo_val.parquet --out-dir data/geo3k_mc

Parity: ``unirl/utils/prepare_dapo_math.py``, ``unirl/utils/prepare_geo3k_mc.py`` (same record layouts, so files written by either load here).
"""

from __future__ import annotations

import argparse
import io
import json
import os
from typing import Any, Dict, Iterable, Iterator, List, Optional

BOXED_REQUEST = "\n\nLet's think step by step and output the final answer within \\boxed{}."
LETTERS = "ABCDEFGH"


# ------------------------------------------------------------------------------------------------ reading
def read_rows(source: str) -> Iterator[Dict[str, Any]]:
    if source.startswith("hub:"):
        try:
            from datasets import load_dataset
        except ImportError as e:  # pragma: no cover
            raise SystemExit(f"{source}: hub sources need the `datasets` package ({e}); pass a local .parquet / .jsonl file instead")
        ident, _, split = source[4:].partition(":")
        yield from load_dataset(ident, split=split or "train")
        return
    if source.endswith(".parquet"):
        import pyarrow.parquet as pq

        yield from pq.read_table(source).to_pylist()
        return
    with open(source) as f:
        for line in f:
            if line.strip():
                yield json.loads(line)


def _first(row: Dict[str, Any], keys: Iterable[str]) -> Any:
    for k in keys:
        if row.get(k) is not None:
            return row[k]
    return None


# ------------------------------------------------------------------------------------------------ math
def math_prompt(row: Dict[str, Any], request_boxed: bool) -> str:
    p = row.get("prompt")
    if isinstance(p, (list, tuple)) and p:  # chat format: the last message is the user's
        last = p[-1]
        text = last.get("content", "") if isinstance(last, dict) else str(last)
    elif isinstance(p, str):
        text = p
    else:
        text = _first(row, ("question", "problem", "Problem", "Question")) or ""
    text = str(text).strip()
    if request_boxed and text and "\\boxed" not in text:
        text += BOXED_REQUEST
    return text


def math_answer(row: Dict[str, Any]) -> Optional[str]:
    for holder, key in (("reward_model", "ground_truth"), ("extra_info", "answer")):
        h = row.get(holder)
        if isinstance(h, dict) and h.get(key) is not None:
            return str(h[key]).strip()
    a = _first(row, ("answer", "Answer", "solution", "final_answer", "gt"))
    return None if a is None else str(a).strip()


def write_math(sources: List[str], out_path: str, request_boxed: bool) -> int:
    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    n = 0
    with open(out_path, "w") as f:
        for src in sources:
            for row in read_rows(src):
                prompt, answer = math_prompt(row, request_boxed), math_answer(row)
                if prompt and answer is not None:  # a row without a checkable answer cannot be rewarded by rule
                    f.write(json.dumps({"prompt": prompt, "metadata": {"answer": answer}}, ensure_ascii=False) + "\n")
                    n += 1
    return n


# ------------------------------------------------------------------------------------------------ multiple choice with a diagram
def mc_prompt(problem: str, choices: List[str]) -> str:
    body = str(problem or "").replace("<image>", "").strip()  # the diagram travels as a media reference, not inline
    lines = "\n".join(f"{LETTERS[i]}) {c}" for i, c in enumerate(choices))
    return f"Look at the geometry diagram. {body}\n\n{lines}\n\nAnswer with the letter only."


def mc_letter(row: Dict[str, Any], choices: List[str]) -> Optional[str]:
    for k in ("ground_truth", "answer_letter", "correct"):
        v = row.get(k)
        if v is not None and str(v).strip()[:1].upper() in LETTERS[: len(choices)]:
            return str(v).strip()[:1].upper()
    a = row.get("answer")
    if a is not None:
        for i, c in enumerate(choices):
            if str(c).strip() == str(a).strip():
                return LETTERS[i]
    return None


def _save_image(img: Any, path: str) -> None:
    """``img``: a PIL image, raw encoded bytes, a ``{"bytes": ...}`` / ``{"path": ...}`` record (parquet image columns) or a file path."""
    from PIL import Image

    if isinstance(img, dict):
        img = img.get("bytes") if img.get("bytes") is not None else img.get("path")
    if isinstance(img, (bytes, bytearray)):
        img = Image.open(io.BytesIO(img))
    elif isinstance(img, str):
        img = Image.open(img)
    img.convert("RGB").save(path)


def write_mc(source: str, split: str, out_path: str, images_dir: str) -> int:
    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    os.makedirs(images_dir, exist_ok=True)
    rel = os.path.relpath(images_dir, os.path.dirname(os.path.abspath(out_path)))
    n = 0
    with open(out_path, "w") as f:
        for idx, row in enumerate(read_rows(source)):
            choices = [str(c) for c in (row.get("choices") or [])]
            problem = _first(row, ("problem", "question"))
            images = row.get("images") or ([row["image"]] if row.get("image") is not None else [])
            letter = mc_letter(row, choices)
            if not choices or not problem or not len(images) or letter is None:
                continue
            sid = int(row["id"]) if row.get("id") is not None else idx
            name = f"{split}_{sid}.png"
            _save_image(images[0], os.path.join(images_dir, name))
            f.write(json.dumps({"prompt": mc_prompt(problem, choices), "prompt_id": f"geo3k:{split}:{sid}",
                                "media_refs": [{"modality": "image", "role": "condition", "uri": f"{rel}/{name}"}],
                                "metadata": {"answer": letter, "answer_value": str(row.get("answer", "")).strip(), "choices": choices, "source_id": sid,
                                             "split": split}}, ensure_ascii=False) + "\n")
            n += 1
    return n


# ------------------------------------------------------------------------------------------------ command line
def main(argv: Optional[List[str]] = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    m = sub.add_parser("dapo-math")
    m.add_argument("--train", nargs="+", default=["hub:BytedTsinghua-SIA/DAPO-Math-17k:train"])
    m.add_argument("--eval", nargs="*", default=["hub:Maxwell-Jia/AIME_2024:train", "hub:yentinglin/aime_2025:train"])
    m.add_argument("--out-dir", default="data/dapo_math")
    m.add_argument("--request-boxed", action="store_true", help="append the \\boxed{} request to prompts that lack one")
    g = sub.add_parser("geo3k-mc")
    g.add_argument("--train", default="hub:xyliu6/geometry3k:train")
    g.add_argument("--val", default="hub:xyliu6/geometry3k:validation")
    g.add_argument("--test", default="", help="optional third split")
    g.add_argument("--out-dir", default="data/geo3k_mc")
    a = ap.parse_args(argv)
    if a.cmd == "dapo-math":
        n = write_math(a.train, os.path.join(a.out_dir, "train.jsonl"), a.request_boxed)
        print(f"train.jsonl: {n} problems")
        if a.eval:
            n = write_math(a.eval, os.path.join(a.out_dir, "aime_eval.jsonl"), a.request_boxed)
            print(f"aime_eval.jsonl: {n} problems")
    else:
        images = os.path.join(a.out_dir, "images")
        for split, src in (("train", a.train), ("val", a.val), ("test", a.test)):
            if src:
                print(f"{split}.jsonl: {write_mc(src, split, os.path.join(a.out_dir, split + '.jsonl'), images)} problems")


if __name__ == "__main__":
    main()
