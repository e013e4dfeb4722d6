"""
Flagship models: builders (RF module trees with checkpoint-compatible parameter names), their ``train_step`` /
``forward_step`` functions, and the fused packed-row execution paths for B200.

- :mod:`conformer_ctc`: Conformer encoder + CTC (12 x 512, 8 heads, FFN 2048, conv kernel 32, conv2d subsampling x6)
- :mod:`blstm_ctc`: 6 x BLSTM(1024) with max-pool time reduction + CTC; :mod:`blstm_12ax` the small CPU task
- :mod:`conformer_aed`: Conformer encoder + Transformer decoder (label-smoothed CE + auxiliary CTC), beam search
- :mod:`transformer_mt`: Transformer-base encoder-decoder for translation
"""
