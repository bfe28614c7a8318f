"""vLLM plugin surface: platform class, patch helper, NVML queries against a fake, registries, entry points."""
import importlib
import sys
import types

import numpy as np
import pytest
import torch

from vllm_metax_b200.patch import utils as pu
from vllm_metax_b200.utils import nvml


# ----------------------------------------------------------------------------- patch helper
@pytest.fixture
def target_module():
    m = types.ModuleType("b200_patch_target")

    def f(x):
        return x + 1

    class C:
        def method(self, x):
            return x * 2

        @staticmethod
        def smethod(x):
            return x - 1

        @property
        def prop(self):
            return "orig"

    m.f, m.C = f, C
    sys.modules[m.__name__] = m
    yield m
    for rec in pu.applied():
        if rec.module == m.__name__:
            pu.revert(rec.module, rec.path)
    del sys.modules[m.__name__]


def test_patch_module_attr_and_double_patch_guard(target_module):
    @pu.patch("b200_patch_target")
    def f(x):
        return x + 100

    assert target_module.f(1) == 101 and pu.is_patched("b200_patch_target", "f")
    assert getattr(target_module.f, pu.MARKER) == ("b200_patch_target", "f")
    assert getattr(target_module.f, pu.ORIGINAL)(1) == 2
    with pytest.raises(RuntimeError):
        pu.apply_patch("b200_patch_target", "f", lambda x: x)
    pu.revert("b200_patch_target", "f")
    assert target_module.f(1) == 2


def test_patch_class_members_keep_descriptor_kind(target_module):
    @pu.patch("b200_patch_target", "C.method")
    def method(self, x):
        return x * 3

    @pu.patch("b200_patch_target", "C.smethod")
    def smethod(x):
        return x - 10

    @pu.patch("b200_patch_target", "C.prop")
    def prop(self):
        return "patched"

    c = target_module.C()
    assert c.method(2) == 6 and target_module.C.smethod(1) == -9 and c.prop == "patched"
    assert isinstance(target_module.C.__dict__["smethod"], staticmethod)
    assert isinstance(target_module.C.__dict__["prop"], property)
    for path in ("C.method", "C.smethod", "C.prop"):
        pu.revert("b200_patch_target", path)
    assert c.method(2) == 4 and c.prop == "orig"


def test_patch_missing_attr_and_missing_module(target_module):
    with pytest.raises(AttributeError):
        pu.apply_patch("b200_patch_target", "nope", lambda: 0)
    pu.apply_patch("b200_patch_target", "nope", lambda: 7, allow_new=True)
    assert target_module.nope() == 7
    pu.revert("b200_patch_target", "nope")
    assert not hasattr(target_module, "nope")

    @pu.patch("module_that_does_not_exist_b200")
    def g():
        return 1
    assert g() == 1


# ----------------------------------------------------------------------------- spec-decode batch order
def test_spec_decode_batch_order_and_swaps():
    from vllm_metax_b200.patch.performance.speculative_decode_perf import plan_order, swaps_for

    #            prefill  decode(q=3) extend  decode(q=1) decode(q=3) long-extend
    sched = np.array([50, 3, 2, 1, 3, 40])
    computed = np.array([0, 20, 5, 9, 12, 30])
    prompt = np.array([50, 10, 30, 8, 8, 100])
    order, sizes = plan_order(sched, computed, prompt, decode_threshold=4)
    assert sizes == {"decode": 3, "short_extend": 1, "long_extend": 1, "prefill": 1}
    assert order.tolist() == [3, 1, 4, 2, 5, 0]        # decodes sorted by query length, stable
    arr = list(range(6))
    for i, j in swaps_for(order):
        arr[i], arr[j] = arr[j], arr[i]
    assert arr == order.tolist()
    assert swaps_for(np.arange(4)) == []


# ----------------------------------------------------------------------------- NVML against a fake
class FakeNvml:
    NVML_CLOCK_SM, NVML_CLOCK_MEM = 1, 2
    NVML_P2P_CAPS_INDEX_NVLINK, NVML_P2P_STATUS_OK = 2, 0
    NVML_NVLINK_MAX_LINKS = 18

    def __init__(self, n=4, broken_pair=None):
        self.n, self.broken, self.inits = n, broken_pair, 0

    def nvmlInit(self):
        self.inits += 1

    def nvmlShutdown(self):
        self.inits -= 1

    def nvmlDeviceGetCount(self):
        return self.n

    def nvmlDeviceGetHandleByIndex(self, i):
        if i >= self.n:
            raise RuntimeError("bad index")
        return i

    def nvmlDeviceGetName(self, h):
        return b"NVIDIA B200"

    def nvmlDeviceGetUUID(self, h):
        return f"GPU-{h:04d}"

    def nvmlDeviceGetCudaComputeCapability(self, h):
        return (10, 0)

    def nvmlDeviceGetMemoryInfo(self, h):
        return types.SimpleNamespace(total=183359 << 20, used=1 << 30)

    def nvmlDeviceGetPciInfo(self, h):
        return types.SimpleNamespace(busId=f"00000000:{h:02X}:00.0".encode())

    def nvmlDeviceGetNumaNodeId(self, h):
        return h // 2

    def nvmlDeviceGetClockInfo(self, h, kind):
        return 1500 if kind == self.NVML_CLOCK_SM else 3996

    def nvmlDeviceGetMaxClockInfo(self, h, kind):
        return 1965

    def nvmlDeviceGetPowerUsage(self, h):
        return 412000

    def nvmlDeviceGetNvLinkState(self, h, link):
        return 1

    def nvmlDeviceGetP2PStatus(self, a, b, idx):
        return 1 if self.broken and {a, b} == set(self.broken) else 0


def test_nvml_queries_with_fake():
    fake = FakeNvml()
    nvml.set_backend(fake)
    try:
        with nvml.session() as n:
            with nvml.session() as inner:       # nested sessions share one init
                assert fake.inits == 1 and inner.device_count() == 4
            assert n.device_name(0) == "NVIDIA B200" and n.device_capability(1) == (10, 0)
            assert n.device_memory_total(0) == 183359 << 20 and n.device_numa_node(3) == 1
            assert n.clocks(0) == {"sm_mhz": 1500, "sm_max_mhz": 1965, "mem_mhz": 3996}
            assert n.nvlink_active_links(0) == 18 and n.fully_connected([0, 1, 2, 3])
            assert len(n.summary()) == 4
        assert fake.inits == 0
        nvml.set_backend(FakeNvml(broken_pair=(1, 2)))
        with nvml.session() as n:
            assert not n.fully_connected([0, 1, 2]) and n.fully_connected([0, 1, 3])
    finally:
        nvml.set_backend(None)


def test_platform_identity_and_backend_selection():
    fake = FakeNvml()
    nvml.set_backend(fake)
    try:
        from vllm_metax_b200 import platform as plat

        P = plat.NvmlB200Platform
        assert P.device_type == "cuda" and P.dispatch_key == "CUDA" and P.dist_backend == "nccl"
        assert str(P._enum).endswith("OOT") or P._enum == "oot"
        assert P.get_device_name(0) == "NVIDIA B200" and tuple(P.get_device_capability(0)) == (10, 0)
        assert P.is_fully_connected([0, 1]) and P.get_device_total_memory(0) == 183359 << 20
        sel = types.SimpleNamespace(use_mla=False, use_sparse=False)
        assert P.get_attn_backend_cls(None, sel).endswith("PagedGQABackend")
        assert P.get_attn_backend_cls(None, types.SimpleNamespace(use_mla=True, use_sparse=False)).endswith("MLABackend")
        assert P.get_attn_backend_cls(None, types.SimpleNamespace(use_mla=True, use_sparse=True)).endswith("MLASparseBackend")
        with pytest.raises(ValueError):
            P.get_attn_backend_cls(types.SimpleNamespace(name="FLASHMLA"), sel)
        assert "fp8" in P.supported_quantization and not P.use_custom_allreduce() and P.opaque_attention_op()
        assert plat._get_backend_priorities(False)[0] == "FLASH_ATTN"
    finally:
        nvml.set_backend(None)


def test_entry_points_resolve():
    import vllm_metax_b200 as pkg

    path = pkg.register()
    mod, cls = path.rsplit(".", 1)
    assert hasattr(importlib.import_module(mod), cls)
    import tomllib

    with open("pyproject.toml", "rb") as f:
        eps = tomllib.load(f)["project"]["entry-points"]
    for group in ("vllm.platform_plugins", "vllm.general_plugins"):
        for target in eps[group].values():
            m, fn = target.split(":")
            assert callable(getattr(importlib.import_module(m), fn))


# ----------------------------------------------------------------------------- vLLM-side registries
def test_registries_with_vllm():
    pytest.importorskip("vllm")
    import vllm_metax_b200 as pkg

    pkg.register_out_of_tree()
    from vllm.model_executor.custom_op import op_registry_oot

    from vllm_metax_b200.registry import custom_ops

    assert {"RMSNorm", "SiluAndMul", "GemmaRMSNorm"} <= set(custom_ops.REGISTERED)
    assert op_registry_oot["RMSNorm"] is custom_ops.REGISTERED["RMSNorm"]
    applied = {(r.module, r.path) for r in pu.applied()}
    assert ("vllm.model_executor.layers.fused_moe.utils", "_int8_quantize") in applied
    # patched int8 quantisation equals the fp32 oracle on CPU
    from vllm.model_executor.layers.fused_moe import utils as fu

    x = torch.randn(4, 64)
    q, s = fu._int8_quantize(x, None, per_act_token=True)
    assert q.dtype == torch.int8 and torch.allclose(q.float() * s, x, atol=float(x.abs().max()) / 100)
    from vllm_metax_b200.models.vllm_registration import VLLM_ARCHITECTURES

    assert "DeepseekV32ForCausalLM" in VLLM_ARCHITECTURES


def test_vllm_backend_metadata_split():
    from vllm_metax_b200.vllm_backends import PagedGQABackend, split_decodes_and_prefills

    qsl = torch.tensor([0, 1, 2, 3, 10, 30])
    assert split_decodes_and_prefills(qsl, 1) == (3, 3)
    assert split_decodes_and_prefills(qsl, 8) == (4, 10)
    assert PagedGQABackend.get_kv_cache_shape(10, 64, 8, 128) == (10, 2, 64, 8, 128)


# ----------------------------------------------------------------------------- all2all packing
def test_pack_unpack_routing_roundtrip():
    from vllm_metax_b200.parallel.all2all import pack_routing, unpack_routing

    w = torch.rand(5, 8)
    ids = torch.randint(0, 256, (5, 8), dtype=torch.int32)
    sc = torch.rand(5, 3)
    packed = pack_routing(w, ids, sc)
    assert packed.shape == (5, 19) and packed.dtype == torch.float32
    w2, ids2, sc2 = unpack_routing(packed, 8)
    assert torch.equal(w2, w) and torch.equal(ids2, ids) and torch.equal(sc2, sc)
    assert unpack_routing(pack_routing(w, ids), 8)[2] is None
