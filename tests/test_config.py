"""Config loading, overrides, coercion, validation, serialisation."""
import pytest

from lset_b200.config import LSETConfig, convert, parse_overrides


def test_defaults_match_reference_surface():
    c = LSETConfig()
    assert c.training.temperature == 0.02 and c.training.scheduler == "cosine"
    assert c.kernels.fused_layernorm is False and c.distributed.dp_size == 1
    assert set(c.to_dict()) >= {"model", "data", "training", "packing", "grad_cache", "compile",
                                "cuda_graph", "kernels", "attention", "activation_checkpoint",
                                "distributed", "lora", "qlora", "fp8", "checkpoint", "logging", "eval"}


def test_yaml_roundtrip_and_unknown_keys(tmp_path):
    p = tmp_path / "c.yaml"
    p.write_text("model:\n  path: /m\ntraining:\n  lr: '3e-5'\n  bogus: 1\nnope:\n  a: 1\n"
                 "training2: 5\n")
    c = LSETConfig.from_yaml(p)
    assert c.model.path == "/m" and c.training.lr == pytest.approx(3e-5)
    out = tmp_path / "o" / "d.yaml"
    c.to_yaml(out)
    assert LSETConfig.from_yaml(out).training.lr == pytest.approx(3e-5)


def test_overrides_and_coercion():
    c = LSETConfig()
    ov = parse_overrides(["--config", "x.yaml", "--training.lr", "1e-4", "--packing.enabled",
                          "--training.matryoshka_dims", "64,128", "--training.top_k", "none",
                          "--lora.targets", "q_proj, v_proj", "--distributed.dp_size", "4"])
    c.apply_overrides(ov)
    assert c.training.lr == 1e-4 and c.packing.enabled is True
    assert c.training.matryoshka_dims == [64, 128] and c.training.top_k is None
    assert c.lora.targets == ["q_proj", "v_proj"] and c.distributed.dp_size == 4
    with pytest.raises(ValueError):
        c.apply_overrides([("training", "1")])
    with pytest.raises(ValueError):
        c.apply_overrides([("nosuch.x", "1")])
    with pytest.raises(ValueError):
        c.apply_overrides([("training.nosuch", "1")])
    assert convert("yes", bool) is True and convert("0", bool) is False


@pytest.mark.parametrize("setup", [
    lambda c: (setattr(c.cuda_graph, "enabled", True), setattr(c.packing, "enabled", True)),
    lambda c: (setattr(c.qlora, "enabled", True), setattr(c.distributed, "tp_size", 2)),
    lambda c: (setattr(c.fp8, "enabled", True), setattr(c.lora, "enabled", True)),
    lambda c: (setattr(c.cuda_graph, "enabled", True), setattr(c.compile, "enabled", True)),
    lambda c: (setattr(c.cuda_graph, "enabled", True), setattr(c.grad_cache, "enabled", True)),
])
def test_validate_rejects(setup):
    c = LSETConfig()
    setup(c)
    with pytest.raises(ValueError):
        c.validate()


def test_yaml_list_fields_accept_lists_and_comma_strings(tmp_path):
    from lset_b200.config import LSETConfig

    f = tmp_path / "c.yaml"
    f.write_text("training:\n  matryoshka_dims: [64, 128]\neval:\n  tasks: STSBenchmark,SICK-R\n")
    c = LSETConfig.from_yaml(f)
    assert c.training.matryoshka_dims == [64, 128] and c.eval.tasks == ["STSBenchmark", "SICK-R"]
    f.write_text("training:\n  matryoshka_dims: 64,128\n")
    assert LSETConfig.from_yaml(f).training.matryoshka_dims == [64, 128]
