import os

import pytest

from arcticinference_b200 import envs, plugin
from arcticinference_b200.patching import ArcticPatch


@pytest.fixture
def classes():
    class Target:
        def my_method(self):
            return "original"

        @classmethod
        def my_classmethod(cls):
            return "original classmethod"

    class Derived(Target):
        def my_method(self):
            return super().my_method() + " derived"

    return Target, Derived


def test_patch_adds_and_replaces(classes):
    Target, Derived = classes

    class P(ArcticPatch[Target]):
        new_field = "new field"

        def new_method(self):
            return "new method"

        def my_method(self):
            return self.__class__.__name__

    P.apply_patch()
    t = Target()
    assert t.new_field == "new field" and t.new_method() == "new method"
    assert t.my_method() == "Target" and Derived().my_method() == "Derived derived"
    assert "_arctic_patches" in Target.__dict__
    assert Target._arctic_patches["new_method"] is P and Target._arctic_patches["my_method"] is P


def test_double_patch_is_refused(classes):
    Target, _ = classes

    class A(ArcticPatch[Target]):
        def my_method(self):
            return "a"

    class B(ArcticPatch[Target]):
        def my_method(self):
            return "b"

    A.apply_patch()
    with pytest.raises(ValueError, match="is already patched by"):
        B.apply_patch()


def test_classmethods_rebind_to_caller(classes):
    Target, Derived = classes

    class P(ArcticPatch[Target]):
        @classmethod
        def my_classmethod(cls):
            return "patched classmethod for %s" % cls.__name__

    P.apply_patch()
    assert Target.my_classmethod() == "patched classmethod for Target"
    assert Derived.my_classmethod() == "patched classmethod for Derived"


def test_special_attrs_not_patched(classes):
    Target, _ = classes
    doc, mod = Target.__doc__, Target.__module__

    class P(ArcticPatch[Target]):
        """patch doc"""
        x = 1

    P.apply_patch()
    assert Target.__doc__ == doc and Target.__module__ == mod and Target.x == 1
    assert "__doc__" not in Target._arctic_patches


def test_patch_needs_target():
    class P(ArcticPatch):
        pass

    with pytest.raises(TypeError):
        P.apply_patch()


def test_envs_are_lazy(monkeypatch):
    monkeypatch.delenv("ARCTIC_INFERENCE_ENABLED", raising=False)
    assert envs.ARCTIC_INFERENCE_ENABLED is False
    assert envs.arctic_inference_effective_enabled() is False
    assert envs.arctic_inference_effective_enabled({"ARCTIC_INFERENCE_ENABLED": "1"}) is True
    monkeypatch.setenv("ARCTIC_INFERENCE_ENABLED", "1")
    assert envs.ARCTIC_INFERENCE_ENABLED is True
    monkeypatch.setenv("ARCTIC_FP32_LM_HEAD", "1")
    assert envs.ARCTIC_FP32_LM_HEAD is True
    with pytest.raises(AttributeError):
        envs.NOT_A_FLAG


def test_registry_knows_reference_architectures():
    archs = plugin.supported_architectures()
    for a in ("LlamaForCausalLM", "LlamaSwiftKVForCausalLM", "ArcticMLPSpeculatorPreTrainedModel",
              "ArcticLSTMSpeculatorPreTrainedModel", "MLPVariantSpeculatorPreTrainedModel", "BertModel"):
        assert a in archs
    with pytest.raises(KeyError):
        plugin.resolve_model("NopeForCausalLM")
