"""View-synthesis model against the reference's own model on a GPU.

The reference's ``uttt_nvs.models.lvsm_moe.Images2latent3D`` (a verbatim copy under ``baseline/_ref/uttt_nvs``, not part
of this repository's history) runs only on CUDA (its Triton kernels allocate there), so this comparison is a GPU test:
same state dict (the key layouts are identical), same scenes, the reference under bf16 autocast over fp32 parameters
as its trainer runs it, ours with bf16 parameters as its trainer runs it.  Compared: the loss, the rendered target
views and the gradient of the patch-embedding weight.  Skipped when the reference tree is absent.
"""
import copy
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "uttt_nvs", "models")),
                    reason="reference tree (baseline/_ref/uttt_nvs) not present")
@pytest.mark.parametrize("extra", [dict(), dict(use_shared_expert=True, shared_expert_per_layer=True)],
                         ids=["routed pool", "with a per-layer always-on expert"])
def test_view_synthesis_model_matches_the_reference_on_gpu(extra):
    import yaml
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import run_reference as rr
    rr._nvs_stand_ins()                       # easydict / omegaconf / lpips / matplotlib are not installed
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from easydict import EasyDict
    from uttt_nvs.models.lvsm_moe import Images2latent3D
    from uttt_b200.nvs.data import SyntheticScenes
    from uttt_b200.nvs.model import LVSMModel

    with open(os.path.join(REF, "uttt_nvs", "configs", "width", "obj", "uttt_moe_e32a2.yaml")) as fh:
        cfg = yaml.safe_load(fh)
    cfg["model"].update(dim=256, layers=2, image_size=128)
    cfg["model"]["block_config"]["params"].update(num_experts=8, num_active_experts=2, **extra)
    cfg["training"].update(num_views=4, lpips_loss_weight=0.0)
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    ref = Images2latent3D(EasyDict(copy.deepcopy(cfg))).to(dev)
    ours_cfg = copy.deepcopy(cfg)
    ours_cfg["model"]["class_name"] = "uttt_b200.nvs.model.LVSMModel"
    ours = LVSMModel(ours_cfg)
    res = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    ours = ours.to(dev).to(torch.bfloat16)
    ref.train()
    ours.train()
    batch = {k: v.to(dev) for k, v in next(SyntheticScenes(2, 4, 128, seed=3, rank=0, pin=False)).items()}

    with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
        out_r = ref({k: v.clone() for k, v in batch.items()})
    loss_r = out_r["loss_metrics"]["loss"]
    loss_r.backward()
    out_o = ours({k: v.clone() for k, v in batch.items()})
    loss_o = out_o["loss_metrics"]["loss"]
    loss_o.backward()
    torch.cuda.synchronize()

    lr_, lo_ = float(loss_r), float(loss_o)
    assert abs(lr_ - lo_) <= 2e-2 * abs(lr_), (lr_, lo_)
    img_r, img_o = out_r["rendering"].float(), out_o["rendering"].float()
    assert img_r.shape == img_o.shape
    assert float((img_r - img_o).abs().mean()) < 1e-2, float((img_r - img_o).abs().mean())
    # the renderings are not constant images (the comparison above would be empty if they were)
    assert float(img_r.std()) > 1e-3
    g_r = ref.image_tokenizer[1].weight.grad.float().flatten()
    g_o = ours.image_tokenizer[1].weight.grad.float().flatten() if hasattr(ours.image_tokenizer, "__getitem__") \
        else dict(ours.named_parameters())["image_tokenizer.1.weight"].grad.float().flatten()
    cos = float(torch.nn.functional.cosine_similarity(g_r, g_o, dim=0))
    assert cos > 0.9, cos
    assert 0.5 < float(g_o.norm() / g_r.norm()) < 2.0
    if extra.get("use_shared_expert"):
        # the always-on experts' initial weights take the same gradient in both implementations
        g_r = ref.transformer_blocks.shared_expert_w1_list[0].grad.float().flatten()
        g_o = ours.transformer_blocks.shared_expert_w1_list[0].grad.float().flatten()
        assert float(torch.nn.functional.cosine_similarity(g_r, g_o, dim=0)) > 0.9
