"""Dataset preparation: raw tables (parquet / jsonl, the column variants seen in the wild) → the records the loaders read."""
import io
import json

import pyarrow as pa
import pyarrow.parquet as pq

from unirl_b200.data.datasets import load_dataset
from unirl_b200.tools import prepare_data as P


def test_math_tables_to_prompt_answer_records(tmp_path):
    rows = [{"prompt": [{"role": "system", "content": "be brief"}, {"role": "user", "content": "What is 2+2?"}], "reward_model": {"ground_truth": "4", "style": "rule"}},
            {"prompt": [{"role": "user", "content": "Give x. Put it in \\boxed{}."}], "reward_model": {"ground_truth": "7", "style": "rule"}},
            {"prompt": [{"role": "user", "content": "no answer here"}], "reward_model": {"ground_truth": None, "style": "rule"}}]
    pq.write_table(pa.Table.from_pylist(rows), tmp_path / "dapo.parquet")
    (tmp_path / "aime24.jsonl").write_text(json.dumps({"Problem": "Find n.", "Answer": 204}) + "\n")
    (tmp_path / "aime25.jsonl").write_text(json.dumps({"question": "Find m.", "answer": "73"}) + "\n" + json.dumps({"question": "", "answer": "1"}) + "\n")
    P.main(["dapo-math", "--train", str(tmp_path / "dapo.parquet"), "--eval", str(tmp_path / "aime24.jsonl"), str(tmp_path / "aime25.jsonl"),
            "--out-dir", str(tmp_path / "out"), "--request-boxed"])
    train = [json.loads(l) for l in (tmp_path / "out" / "train.jsonl").read_text().splitlines()]
    assert [r["metadata"]["answer"] for r in train] == ["4", "7"]  # the row without a ground truth is dropped
    assert train[0]["prompt"] == "What is 2+2?" + P.BOXED_REQUEST and train[1]["prompt"].count("\\boxed") == 1
    ev = [json.loads(l) for l in (tmp_path / "out" / "aime_eval.jsonl").read_text().splitlines()]
    assert [(r["prompt"].split("\n")[0], r["metadata"]["answer"]) for r in ev] == [("Find n.", "204"), ("Find m.", "73")]
    ds = load_dataset(str(tmp_path / "out" / "train.jsonl"))
    assert len(ds) == 2 and ds[0]["metadata"] == {"answer": "4"} and ds[0]["media"] is None


def test_multiple_choice_with_diagram(tmp_path):
    from PIL import Image

    buf = io.BytesIO()
    Image.new("RGB", (8, 6), (200, 10, 10)).save(buf, format="PNG")
    rows = [{"id": 11, "problem": "<image>Find the angle.", "choices": ["30", "45", "60", "90"], "ground_truth": "C", "answer": "60", "images": [{"bytes": buf.getvalue(), "path": None}]},
            {"id": 12, "problem": "Find x.", "choices": ["1", "2"], "ground_truth": None, "answer": "2", "images": [{"bytes": buf.getvalue(), "path": None}]},
            {"id": 13, "problem": "No picture.", "choices": ["1", "2"], "ground_truth": "A", "answer": "1", "images": []}]
    pq.write_table(pa.Table.from_pylist(rows), tmp_path / "geo.parquet")
    P.main(["geo3k-mc", "--train", str(tmp_path / "geo.parquet"), "--val", "", "--out-dir", str(tmp_path / "geo")])
    recs = [json.loads(l) for l in (tmp_path / "geo" / "train.jsonl").read_text().splitlines()]
    assert [r["metadata"]["answer"] for r in recs] == ["C", "B"]  # the letter given, or found by matching the answer value; the row without a diagram is dropped
    assert recs[0]["prompt"] == "Look at the geometry diagram. Find the angle.\n\nA) 30\nB) 45\nC) 60\nD) 90\n\nAnswer with the letter only."
    assert recs[0]["media_refs"] == [{"modality": "image", "role": "condition", "uri": "images/train_11.png"}]
    ds = load_dataset(str(tmp_path / "geo" / "train.jsonl"))
    row = ds[0]
    assert row["metadata"]["answer"] == "C" and row["metadata"]["prompt_id"] == "geo3k:train:11" and row["metadata"]["choices"] == ["30", "45", "60", "90"]
    assert len(row["media"]) == 1 and row["media"][0].kind == "image" and Image.open(row["media"][0].path).size == (8, 6)
