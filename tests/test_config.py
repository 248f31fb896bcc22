import json

import pytest

import brolm_b200 as bb
from brolm_b200.config import architecture_of, registered_architectures
from tests.helpers import TINY_A, TINY_B


def test_defaults_are_gemma_2_2b():
    c = bb.Gemma2Config.from_json_text("{}")
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (256000, 2304, 9216, 26)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (8, 4, 256)
    assert c.sliding_window == 4096 and c.query_pre_attn_scalar == 256.0 and c.tie_word_embeddings
    assert c.q_dim == 2048 and c.kv_dim == 1024
    assert [c.is_sliding(i) for i in range(4)] == [True, False, True, False]


def test_keys_are_read_and_null_means_default():
    c = bb.Gemma2Config.from_json_text(json.dumps({**TINY_B, "rope_theta": None, "unknown_key": 3}))
    assert c.hidden_size == 96 and c.head_dim == 32 and c.rope_theta == 10000.0
    assert c.query_pre_attn_scalar == 24.0 and c.rms_norm_eps == 1e-5


def test_query_scalar_may_differ_from_head_dim():
    c = bb.Gemma2Config.from_json_text(json.dumps({"head_dim": 128, "query_pre_attn_scalar": 144}))
    assert c.query_pre_attn_scalar == 144.0


def test_layer_types_win_over_parity():
    c = bb.Gemma2Config.from_json_text(json.dumps({**TINY_A, "layer_types": ["full_attention", "sliding_attention"]}))
    assert [c.is_sliding(0), c.is_sliding(1)] == [False, True]
    with pytest.raises(bb.ConfigError):
        bb.Gemma2Config.from_json_text(json.dumps({**TINY_A, "layer_types": ["full_attention"]}))


@pytest.mark.parametrize("bad", [{"hidden_size": 0}, {"num_attention_heads": 6, "num_key_value_heads": 4},
                                 {"head_dim": 7}, {"sliding_window": 0}, {"rms_norm_eps": 0.0},
                                 {"query_pre_attn_scalar": -1}, {"hidden_size": "wide"}, {"vocab_size": 3.5},
                                 {"hidden_activation": "relu"}, {"tie_word_embeddings": 1}])
def test_bad_values_are_refused(bad):
    with pytest.raises(bb.ConfigError):
        bb.Gemma2Config.from_json_text(json.dumps(bad))


def test_malformed_json_and_missing_file(tmp_path):
    with pytest.raises(bb.ConfigError, match="json parse"):
        bb.Gemma2Config.from_json_text("{not json")
    with pytest.raises(bb.ConfigError, match="not a JSON object"):
        bb.Gemma2Config.from_json_text("[1, 2]")
    with pytest.raises(bb.ConfigError, match="cannot open"):
        bb.load_config(str(tmp_path / "nowhere"))


def test_registry_picks_the_model_by_name(tmp_path):
    assert "Gemma2ForCausalLM" in registered_architectures()
    assert architecture_of({"architectures": ["Gemma2ForCausalLM"]}).config_cls is bb.Gemma2Config
    assert architecture_of({"model_type": "gemma2"}).config_cls is bb.Gemma2Config
    with pytest.raises(bb.ConfigError, match="registered"):
        architecture_of({"architectures": ["SomethingElse"]})
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["Gemma2ForCausalLM"], **TINY_A}))
    c = bb.load_config(str(tmp_path))
    assert isinstance(c, bb.Gemma2Config) and c.hidden_size == 64


def test_round_trip_through_to_dict():
    c = bb.Gemma2Config(**TINY_B)
    assert bb.Gemma2Config.from_dict(json.loads(json.dumps(c.to_dict()))) == c


def test_layout_follows_the_configuration():
    from brolm_b200.models.gemma2 import gemma2_layout
    c = bb.Gemma2Config(**TINY_B)
    lay = gemma2_layout(c)
    assert len(lay.blocks) == 3 and [s.block for s in lay.schedule] == [0, 1, 2]
    assert [b.mixer.args["window"] for b in lay.blocks] == [16, None, 16]
    assert lay.blocks[0].mixer.args["scale"] == 24 ** -0.5 and lay.head.softcap == 15.0
    assert lay.embedding.scale == pytest.approx(96 ** 0.5)


def test_absent_and_null_keys_read_as_in_the_reference(tmp_path):
    """The same document through wlejon/brolm's own JSON reader (tests/golden/json_defaults.cpp) and
    through Gemma2Config: absent and null keys give the defaults, present ones their values."""
    import os
    import shutil
    import subprocess
    here = os.path.dirname(os.path.abspath(__file__))
    expected = open(os.path.join(here, "golden", "json_defaults.expected")).read()
    # with a checkout of wlejon/brolm at hand ($BROLM_REFERENCE) the program is built again from its header
    ref_include = os.path.join(os.environ.get("BROLM_REFERENCE", ""), "include")
    if shutil.which("g++") and os.path.exists(os.path.join(ref_include, "brolm", "detail", "json.h")):
        exe = str(tmp_path / "json_defaults")
        subprocess.check_call(["g++", "-std=c++20", "-I", ref_include, os.path.join(here, "golden", "json_defaults.cpp"),
                               "-o", exe])
        assert subprocess.check_output([exe], text=True) == expected      # the committed output is still the reader's
    doc = ('{"hidden_size": 96, "head_dim": null, "rms_norm_eps": 1e-5, "tie_word_embeddings": false, '
           '"vocab_size": 512.0, "rope_theta": null}')
    c = bb.Gemma2Config.from_json_text(doc)
    got = {"hidden_size": c.hidden_size, "head_dim": c.head_dim, "num_hidden_layers": c.num_hidden_layers,
           "vocab_size": c.vocab_size, "tie_word_embeddings": int(c.tie_word_embeddings)}
    want = dict(line.split() for line in expected.splitlines())
    for key, value in got.items():
        assert int(want[key]) == value, key
    assert abs(float(want["rms_norm_eps"]) - c.rms_norm_eps) < 1e-12 and float(want["rope_theta"]) == c.rope_theta
