"""
Importing parameters of models from other toolkits into RF modules:
``torch_nn`` (torch.nn.Linear / Conv1d / LayerNorm), ``hf_llama`` (HuggingFace Llama -> TransformerDecoder),
``espnet_e_branchformer`` (ESPnet E-Branchformer layer -> EBranchformerLayer).
"""
