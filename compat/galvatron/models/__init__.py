"""``galvatron.models`` under its reference name: one sub-package per model directory of the reference
(``llama_hf, llama_fa, gpt_hf, gpt_fa, bert_hf, vit_hf, T5, swin``) with the modules user programs import from
(``<X>Model_hybrid_parallel``, ``<X>Model_checkpoint``, ``arguments``, ``dataloader``, ``meta_configs``), every name bound
to its counterpart in ``hetu_galvatron_b200`` (see ``hetu_galvatron_b200/models/reference_names.py``)."""
from hetu_galvatron_b200.models.reference_names import install as _install

globals().update(_install(__name__))
