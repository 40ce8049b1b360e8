"""How parts, blocks and cache groups are found and built, without a GPU: nested part specs, families of
one's own, a block with other parts than the pre-norm block's, sizes no kernel takes, and a cache need
with a group class of its own."""
from dataclasses import dataclass

import pytest
import torch

from conftest import TINY_A
from gpullama3.java_b200.cache import (CacheError, CacheFull, PagedGroup, SequenceCache, register_cache_group,
                                       unregister_cache_group)
from gpullama3.java_b200.config import ConfigError, LayerSpec, PartSpec, config_from_dict
from gpullama3.java_b200.parts import (Block, Norm, Part, PartRegistryError, RMSNorm, RotaryPositionEncoding,
                                       build_block, build_part, register_block, register_part, registered, unregister)


class Holder(Part):
    def __init__(self, inner, others=(), named=None, number=0):
        self.inner, self.others, self.named, self.number = inner, others, named or {}, number

    def children(self):
        return {"inner": self.inner}


def test_part_specs_nest_under_any_key():
    norm = PartSpec("norm", "rmsnorm", {"dim": 8, "eps": 1e-3})
    rope = PartSpec("position", "rope", {"head_dim": 16, "theta": 100.0})
    register_part("test_family", "holder", Holder)
    try:
        assert "holder" in registered("test_family")
        h = build_part(PartSpec("test_family", "holder", {"inner": norm, "others": [rope, norm], "named": {"a": rope},
                                                        "number": 3}))
        assert isinstance(h.inner, RMSNorm) and h.inner.eps == 1e-3 and h.number == 3
        assert isinstance(h.others[0], RotaryPositionEncoding) and isinstance(h.others[1], RMSNorm)
        assert isinstance(h.named["a"], RotaryPositionEncoding)
        with pytest.raises(PartRegistryError, match="already registered"):
            register_part("test_family", "holder", Holder)
    finally:
        unregister("test_family", "holder")
    with pytest.raises(PartRegistryError, match="unknown norm kind 'layernorm'; registered: rmsnorm"):
        build_part(PartSpec("norm", "layernorm", {}))
    with pytest.raises(PartRegistryError, match="unknown part family"):
        build_part(PartSpec("nothing", "x", {}))


class MixerOnlyBlock(Block):
    """A block with other parts than the pre-norm block's: no feed-forward, a norm after the mixer."""

    def __init__(self, mixer, after):
        super().__init__(mixer=mixer, after=after)


def test_a_block_names_its_own_parts_and_nested_parameters_get_paths():
    from gpullama3.java_b200.engine.model import CausalLM

    register_block("test_mixer_only", MixerOnlyBlock)
    try:
        cfg = config_from_dict(TINY_A)
        base = cfg.layer_specs()[0]
        spec = LayerSpec("test_mixer_only", {"mixer": base.parts["mixer"], "after": base.parts["mixer_norm"]})
        b = build_block(spec)
        assert sorted(b.children()) == ["after", "mixer"] and isinstance(b.after, Norm)
        assert b.cache_need() == b.mixer.cache_need()
        with pytest.raises(PartRegistryError, match="does not take the parts"):
            build_block(LayerSpec("test_mixer_only", dict(base.parts)))          # pre-norm parts to this block ...
        with pytest.raises(PartRegistryError, match="does not take the parts"):
            build_block(LayerSpec("pre_norm", {"mixer": base.parts["mixer"]}))   # ... and too few for pre-norm
    finally:
        unregister("block", "test_mixer_only")
    model = CausalLM(cfg, torch.float32, "cpu")
    paths = model.named_parts()
    assert "layers.1.mixer.position" in paths and "layers.0.feed_forward_norm" in paths
    assert set(model.parameter_specs()) == set(cfg.tensor_names())


@pytest.mark.parametrize("change, match", [({"head_dim": 72}, "steps of 16"), ({"head_dim": 272}, "up to 256"),
                                           ({"head_dim": 8}, "steps of 16")])
def test_head_sizes_no_kernel_takes_are_refused_when_the_model_is_built(change, match):
    from gpullama3.java_b200.engine.model import CausalLM

    cfg = config_from_dict(dict(TINY_A, **change))      # the configuration itself only asks for an even head size
    with pytest.raises(ConfigError, match=match):
        CausalLM(cfg, torch.float32, "cpu")


def test_optional_tensor_names_come_from_the_configuration():
    assert config_from_dict(TINY_A).optional_tensor_names() == {"lm_head.weight"}          # tied
    assert config_from_dict(dict(TINY_A, tie_word_embeddings=False)).optional_tensor_names() == set()


@dataclass(frozen=True)
class RowNeed:
    """One row of ``width`` numbers per position."""
    width: int


class RowGroup(PagedGroup):
    def __init__(self, need, entries, sizes):
        super().__init__(need, entries, sizes)
        self.rows_data = torch.zeros((len(self.entries), self.pool.n_pages, 64, need.width), dtype=sizes.dtype,
                                     device=sizes.device)

    def view(self, entry):
        return ("rows", self.index, self.rows_data[self.entry_pos[entry]])

    def bytes_per_token(self):
        return len(self.entries) * self.need.width * self.rows_data.element_size()


def test_a_cache_need_of_ones_own_brings_its_group_class():
    from gpullama3.java_b200.cache import KVCacheNeed, StateNeed

    with pytest.raises(TypeError, match="no cache group is registered"):
        SequenceCache({0: RowNeed(5)}, max_tokens=256, device="cpu")
    register_cache_group(RowNeed, RowGroup)
    try:
        with pytest.raises(CacheError):
            register_cache_group(RowNeed, RowGroup)
        c = SequenceCache({0: RowNeed(5), 1: KVCacheNeed(1, 16), 2: RowNeed(5), 3: StateNeed((2,)), 4: RowNeed(7)},
                          max_tokens=64 * 4, max_slots=3, dtype=torch.float32, device="cpu")
        assert len(c.paged_groups) == 3 and len(c.slot_groups) == 1      # RowNeed(5) x2, KV, RowNeed(7); state
        kind, gi, data = c.view(2)
        assert kind == "rows" and tuple(data.shape) == (4, 64, 5) and c.paged_groups[gi].entries == [0, 2]
        assert c.bytes_per_token() == (2 * 5 + 7) * 4 + 2 * 16 * 4
        a, b = c.acquire(), c.acquire()
        c.reserve([(a, 100), (b, 64)])
        c.commit(a, 100)
        c.commit(b, 64)
        assert [len(r) for r in c.page_rows(gi, [a, b])] == [2, 1]
        with pytest.raises(CacheFull):
            c.reserve([(b, 65)])                      # 2 more pages, 1 is free: nothing changes
        assert len(c.page_rows(gi, [b])[0]) == 1
        c.check_invariants()
        c.release(a)
        c.reserve([(b, 65)])
        c.check_invariants()
        c.release(b)
        assert all(g.pool.n_free == g.pool.n_pages for g in c.paged_groups)
    finally:
        unregister_cache_group(RowNeed)
