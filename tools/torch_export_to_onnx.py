#!/usr/bin/env python3
"""
Export the forward computation of a config's model to ONNX: ``forward_step`` is traced over a dummy batch built from
``extern_data``; inputs are the extern_data tensors and their length vectors, outputs the tensors marked with ``mark_as_output``.
Needs the ``onnx`` package (``torch.onnx``). Models that take the fused CUDA paths must be exported on the CPU (the kernels are
not ONNX ops).

    tools/torch_export_to_onnx.py my.config model.010.pt out.onnx

(reference: tools/torch_export_to_onnx.py)
"""

import argparse
import torch
import _setup_returnn_env  # noqa: F401
from returnn_b200 import __main__ as rnn
from returnn_b200 import frontend as rf
from returnn_b200.tensor import Tensor, TensorDict, batch_dim
from returnn_b200.torch.data.extern_data import extern_data_template_from_config_opts


class _Wrapper(torch.nn.Module):
    def __init__(self, model, forward_step, template: TensorDict, keys):
        super().__init__()
        self.model_pt = model if isinstance(model, torch.nn.Module) else rf.rf_module_to_pt_module(model)
        self.model, self.forward_step, self.template, self.keys = model, forward_step, template, keys

    def forward(self, *raws):
        ed = TensorDict()
        it = iter(raws)
        batch_dim.dyn_size_ext = None
        for k in self.keys:
            t = self.template.data[k].copy_template()
            t._raw_tensor = next(it)
            for d in t.dims:
                if d.is_dynamic() and not d.is_batch_dim():
                    d.dyn_size_ext = Tensor("%s:len" % k, dims=[batch_dim], dtype="int32", raw_tensor=next(it))
            ed.data[k] = t
        rf.init_forward_step_run_ctx(expected_outputs=None)
        self.forward_step(model=self.model, extern_data=ed)
        outs = rf.get_run_ctx().outputs
        return tuple(v.raw_tensor for v in outs.data.values())


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("config")
    ap.add_argument("checkpoint")
    ap.add_argument("out_onnx")
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--time", type=int, default=50)
    args = ap.parse_args()
    try:
        import onnx  # noqa: F401
    except ImportError:
        raise SystemExit("the onnx package is not installed: cannot export")
    rnn.init(config_filename=args.config, command_line_options=["++task", "nop", "++device", "cpu", "++load", args.checkpoint[:-3] if args.checkpoint.endswith(".pt") else args.checkpoint])
    config = rnn.config
    template = extern_data_template_from_config_opts(config.typed_value("extern_data"))
    get_model, forward_step = config.typed_value("get_model"), config.typed_value("forward_step")
    model = get_model(epoch=1, step=0)
    ck = torch.load(args.checkpoint, map_location="cpu")
    pt = model if isinstance(model, torch.nn.Module) else rf.rf_module_to_pt_module(model)
    pt.load_state_dict(ck["model"])
    pt.eval()
    keys = [k for k, v in template.data.items() if v.available_for_inference and v.dtype != "string"]
    raws, names = [], []
    for k in keys:
        t = template.data[k]
        shape = [args.batch if d.is_batch_dim() else (d.dimension if d.dimension is not None else args.time) for d in t.dims]
        raws.append(torch.randint(0, t.sparse_dim.dimension, shape, dtype=torch.int32) if t.sparse_dim is not None else torch.randn(shape))
        names.append(k)
        if any(d.is_dynamic() and not d.is_batch_dim() for d in t.dims):
            raws.append(torch.full((args.batch,), args.time, dtype=torch.int32))
            names.append("%s:seq_len" % k)
    wrapper = _Wrapper(model, forward_step, template, keys)
    with torch.no_grad():
        torch.onnx.export(wrapper, tuple(raws), args.out_onnx, input_names=names, opset_version=17,
                          dynamic_axes={n: {0: "batch", **({1: "time"} if not n.endswith(":seq_len") else {})} for n in names})
    print("exported", args.out_onnx)


if __name__ == "__main__":
    main()
