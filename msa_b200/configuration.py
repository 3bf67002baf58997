"""``MSAConfig``: Qwen3Config plus the ``msa_config`` dictionary with attribute access
(mirror of src/msa/configuration_msa.py:6-53; keys as written by src/utils/resave_model.py:33-50)."""
from transformers.models.qwen3.configuration_qwen3 import Qwen3Config


class DotDict(dict):
    __getattr__ = dict.get
    __setattr__ = dict.__setitem__
    __delattr__ = dict.__delitem__

    def __getstate__(self):
        return dict(self)

    def __setstate__(self, state):
        self.update(state)


MSA_CONFIG_DEFAULTS = dict(
    router_layer_idx="all", aux_loss=False, aux_loss_method="INFONCE", decouple_router=False, rewrite_position=False,
    top_k_docs=2, pooling_kernel_size=2, infonce_loss_temp=0.1, head_reduce_method="max", query_reduce_method="max",
    chunk_reduce_method="max", decouple_pooling_mode="mean")


class MSAConfig(Qwen3Config):
    model_type = "msa"

    def __init__(self, msa_config=None, **kwargs):
        super().__init__(**kwargs)
        if msa_config is not None:
            self.msa_config = msa_config

    def __setattr__(self, name, value):
        if name == "msa_config" and isinstance(value, dict) and not isinstance(value, DotDict):
            value = DotDict(value)
        super().__setattr__(name, value)
