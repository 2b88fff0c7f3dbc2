import pytest
import torch
from dataclasses import dataclass
from typing import List, Optional

from unirl_b200.distributed.tensor.batch import Batch, concat_field, max_field, mean_field, packed_field, shared_field, sum_field
from unirl_b200.distributed.tensor.pytree import infer_batch_size, pytree_cat, pytree_chunk
from unirl_b200.distributed.tensor.transport import TensorMeta, TensorRef
from unirl_b200.distributed.utils import Broadcast
from unirl_b200.types import (ARSamplingParams, RolloutReq, RolloutResp, RolloutTrack, TextSegment, TextTokenCondition, Texts, Trajectory,
                              TrajectoryBuilder, compute_trajectory_positions, LatentSegment, DiffusionSamplingParams, RolloutInputs)


@dataclass
class Toy(Batch):
    x: Optional[torch.Tensor] = concat_field(default=None)
    names: List[str] = concat_field(default_factory=list)
    sched: Optional[torch.Tensor] = shared_field(default=None)
    tok: Optional[torch.Tensor] = packed_field(default=None)
    wall: float = max_field(default=0.0)
    total: float = sum_field(default=0.0)
    avg: float = mean_field(default=0.0)
    extra: dict = concat_field(default_factory=dict)


def make(n, off=0):
    return Toy.pack(x=torch.arange(n * 2.0).view(n, 2) + off, names=[f"s{off + i}" for i in range(n)], sched=torch.ones(3),
                    tok=[torch.full((i + 1,), float(off + i)) for i in range(n)], wall=float(off), total=1.0, avg=float(off),
                    extra={"m": torch.arange(n) + off, "l": list(range(n))})


def test_concat_slice_select_repeat_roundtrip():
    a, b = make(3), make(2, 10)
    c = Toy.concat([a, b])
    assert c.batch_size == 5 and c.names == ["s0", "s1", "s2", "s10", "s11"]
    assert c.cu_seqlens.tolist() == [0, 1, 3, 6, 7, 9]
    assert c.wall == 10.0 and c.total == 2.0 and c.avg == 5.0
    assert torch.equal(c.sched, torch.ones(3))
    s = c.slice(2, 4)
    assert s.names == ["s2", "s10"] and s.cu_seqlens.tolist() == [0, 3, 4] and s.tok.tolist() == [2.0, 2.0, 2.0, 10.0]
    assert s.extra["m"].tolist() == [2, 10] and s.extra["l"] == [2, 0]
    sel = c.select(torch.tensor([4, 0]))
    assert sel.names == ["s11", "s0"] and sel.tok.tolist() == [11.0, 11.0, 0.0]
    rep = a.repeat_interleave(2)
    assert rep.names == ["s0", "s0", "s1", "s1", "s2", "s2"] and rep.lengths.tolist() == [1, 1, 2, 2, 3, 3]
    parts = c.slice(0, 4).chunk(2)
    assert Toy.concat(parts).tok.tolist() == c.slice(0, 4).tok.tolist()
    cl = c.clone()
    cl.x += 1
    assert not torch.equal(cl.x, c.x)
    with pytest.raises(ValueError):
        c.chunk(2)


def test_pack_rejects_mismatched_sizes():
    with pytest.raises(ValueError):
        TextSegment.pack(tokens=[torch.zeros(2), torch.zeros(3)], log_probs=[torch.zeros(2), torch.zeros(2)])


def test_pytree_chunk_cat_and_broadcast():
    payload = ({"a": torch.arange(8).view(4, 2), "meta": torch.arange(3)}, [1, 2, 3, 4], Broadcast([9, 9, 9, 9]), "s", make(4))
    assert infer_batch_size(payload, {}) == 4
    shards = pytree_chunk(payload, 2, 4)
    assert shards[0][0]["a"].shape == (2, 2) and shards[1][0]["meta"].tolist() == [0, 1, 2]
    assert shards[0][2] == [9, 9, 9, 9] and shards[1][1] == [3, 4] and shards[1][4].batch_size == 2
    back = pytree_cat([s[0] for s in shards])
    assert torch.equal(back["a"], payload[0]["a"])
    with pytest.raises(ValueError):
        pytree_chunk(torch.zeros(3, 1), 2, 3)


def test_tensor_meta_slices_on_ref_boundaries():
    refs = [TensorRef(0, 1, (2, 3), torch.float32, "cpu"), TensorRef(1, 1, (4, 3), torch.float32, "cpu")]
    m = TensorMeta.from_refs(refs)
    assert m.batch_size == 6 and m.shape == (6, 3)
    assert m.slice(2, 6).refs == [refs[1]] and m[0:2].refs == [refs[0]]
    cut = m.slice(1, 3)  # a range inside handles becomes windows of them
    assert [(r.owner, r.lo, r.rows) for r in cut.refs] == [(0, 1, 1), (1, 0, 1)] and cut.refs[0].base is refs[0]
    parts = pytree_chunk(m, 2, 6)
    assert [p.batch_size for p in parts] == [2, 4]
    assert pytree_cat(parts).refs == refs


def _track(rewards, groups=2, branch=3):
    req = RolloutReq(sample_ids=[f"p{i}" for i in range(groups)], group_ids=[f"p{i}" for i in range(groups)])
    t = req.make_root_track("ar", branch)
    return t.replace(rewards=torch.tensor(rewards))


def test_advantages_group_global_and_errors():
    t = _track([1.0, 0.0, 0.0, 1.0, 1.0, 1.0])
    adv = t.compute_advantages().advantages
    r = torch.tensor([[1.0, 0, 0], [1, 1, 1]])
    exp = (r - r.mean(1, keepdim=True)) / (r.var(1, unbiased=False, keepdim=True) + 1e-8).sqrt()
    assert torch.allclose(adv, exp.flatten(), atol=1e-6)
    assert torch.allclose(t.compute_advantages(normalize=False).advantages, (r - r.mean(1, keepdim=True)).flatten())
    g = t.compute_advantages(scope="global").advantages
    assert torch.allclose(g, (r.flatten() - r.mean()) / (r.flatten().std() + 1e-8))
    gs = t.compute_advantages(use_global_std=True).advantages
    assert torch.allclose(gs, ((r - r.mean(1, keepdim=True)) / (r.flatten().std() + 1e-8)).flatten())
    bad = t.replace(parent_ids=["p0", "p1", "p0", "p1", "p0", "p1"])
    with pytest.raises(ValueError):
        bad.compute_advantages()


def test_resp_lineage_split_and_reward_propagation():
    req = RolloutReq(sample_ids=["a", "b"], group_ids=["a", "b"], primitives={"text": Texts(texts=["x", "y"])})
    ar = req.make_root_track("ar", 2)
    img = ar.fork_track("ar", "image", 3).replace(rewards=torch.arange(12.0))
    resp = RolloutResp(tracks={"ar": ar, "image": img})
    out = resp.propagate_rewards("mean")
    assert out.tracks["ar"].rewards.tolist() == [1.0, 4.0, 7.0, 10.0]
    assert resp.propagate_rewards("max").tracks["ar"].rewards.tolist() == [2.0, 5.0, 8.0, 11.0]
    parts = out.split()
    assert len(parts) == 2 and parts[1].tracks["image"].batch_size == 6 and parts[1].tracks["ar"].sample_ids == ["b/a0", "b/a1"]
    with pytest.raises(ValueError):
        RolloutResp(tracks={"image": img})
    light = out.metadata_only()
    assert light.tracks["image"].segment is None and light.tracks["image"].rewards is not None


def test_text_condition_concat_pads():
    a = TextTokenCondition(input_ids=torch.ones(2, 3, dtype=torch.long), attention_mask=torch.ones(2, 3, dtype=torch.long))
    b = TextTokenCondition(input_ids=torch.ones(1, 5, dtype=torch.long), attention_mask=torch.ones(1, 5, dtype=torch.long))
    c = TextTokenCondition.concat([a, b])
    assert c.input_ids.shape == (3, 5) and c.attention_mask[0].tolist() == [1, 1, 1, 0, 0]


def test_trajectory_builder_and_positions():
    assert compute_trajectory_positions({0, 2, 4}, 5) == [0, 1, 2, 3, 4, 5] and compute_trajectory_positions({3}, 5) == [3, 4]
    b = TrajectoryBuilder.for_sde_steps({1, 3}, 5)
    for p in range(6):
        b.add(p, torch.full((2, 4), float(p)))
    tr = b.finalize()
    assert tr.stored_positions == [1, 2, 3, 4] and tr.is_selective
    x, y = tr.get_pair(3)
    assert float(x[0, 0]) == 3.0 and float(y[0, 0]) == 4.0
    with pytest.raises(IndexError):
        tr.get_position(0)
    assert Trajectory.from_clean_latents(torch.zeros(2, 4), 6).clean_latents.shape == (2, 4)


def test_latent_segment_keeps_modality_and_sampling_params():
    from unirl_b200.types import make_video_segment, Modality

    s = make_video_segment(latents=torch.zeros(4, 2, 3), indices=torch.tensor([0, 5]))
    assert s.select(torch.tensor([1, 2])).modality is Modality.VIDEO and s.latents_at(5).shape == (4, 3)
    with pytest.raises(KeyError):
        s.latents_at(2)
    p = DiffusionSamplingParams(num_inference_steps=4, sde_indices=[1, 2])
    assert p.resolve_sde_indices(7) == [1, 2]
    assert DiffusionSamplingParams(num_inference_steps=3).resolve_sde_indices(0) == [0, 1, 2]
    with pytest.raises(ValueError):
        DiffusionSamplingParams(sampler_kwargs={"eta": 1})
    inp = RolloutInputs(primitives={"text": Texts(texts=["a", "b"])}, sample_ids=["x", "y"], group_ids=["g0", "g1"], metadata=[None, None]).expand(2)
    assert inp.sample_ids == ["prompt:g0:sample:0", "prompt:g0:sample:1", "prompt:g1:sample:0", "prompt:g1:sample:1"]
