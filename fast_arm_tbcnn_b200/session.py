"""Device-resident graph executor mirroring the reference's ``TBNModel::Session``
(tbn-runtime/include/tbn/runtime/model.hpp:119-1316) for the operators of the CNN configurations.

A graph is a plain dict with the fields of the reference's ``ModelGraph`` (model.hpp:29-35):

    {"inputs": {name: shape}, "outputs": {name: shape}, "inits": {name: ndarray},
     "binary": {names of weight tensors to binarise}, "nodes": [{"op", "name", "inputs", "outputs", "attrs"}]}

Same surface as the reference: ``set_quantization(bool)``, ``set_input(name, array)``, ``run()``,
``get_output(name)``; ``set_input`` checks the shape against the graph (InvalidShapeError there, ValueError
here).  All tensors live in HBM; weights are sign-packed once at construction (the reference caches them on
the first run, model.hpp:127-157).  Every operator runs in the CUDA library through its C ABI.

Two numeric modes, selected like the reference's quantisation switch:
  * quantisation off (default) -- "float x binary": y = x * (alpha * sign(w)) in fp32 accuracy, which is what
    the reference computes with quantisation off on the dequantised weights alpha*sign(w);
  * quantisation on -- "TBN mode": activations ternarised at +-0.1, exact integer accumulation,
    (acc + bias) * alpha for Conv and acc + bias for Gemm, bit-equal to the reference Session with
    quantisation on when it is given the dequantised weights.
"""
import numpy as np

from . import capi


class Session:
    def __init__(self, graph, device=None, fuse=True, fast=True, chain=True):
        import torch
        self.torch = torch
        self.graph = graph
        self.L = capi.lib
        self.device = torch.device("cuda", self.L.init(device))
        self.quantization = False
        self.fuse = fuse
        self.fast = fast  # channels-last convolution path where the channel count allows it
        # Layer chaining (float x binary mode): a convolution whose result feeds channels-last convolutions writes the
        # bf16 channels-last form from its epilogue (and skips the fp32 NCHW tensor when nothing else reads it), and
        # those convolutions skip their pre-pass.  Same bits as the unchained execution.
        self.chain = chain and fast
        self.inputs = {}
        self.values = {}
        self.weights = {}
        conv_w = {n["inputs"][1] for n in graph["nodes"] if n["op"] == "Conv"}
        gemm_w = {n["inputs"][1] for n in graph["nodes"] if n["op"] == "Gemm"}
        for name, arr in graph["inits"].items():
            t = torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32)).to(self.device)
            if name in graph["binary"]:
                self.weights[name] = self._pack(t)
            elif name in conv_w:   # float filters: split once into two bf16 terms
                order = capi.CONV_WEIGHTS_TAP_MAJOR if (fast and t.shape[1] % 64 == 0) else capi.CONV_WEIGHTS_REFERENCE
                flat = self.L.permute_filters(t) if order else t.reshape(t.shape[0], -1)
                self.weights[name] = {"shape": tuple(t.shape), "order": order,
                                      "split": self.L.dense_pack(flat, capi.LAYOUT_NK)}
            elif name in gemm_w:   # float Gemm B [K, N]
                self.weights[name] = {"shape": tuple(t.shape), "split": self.L.dense_pack(t, capi.LAYOUT_KN)}
            else:
                self.weights[name] = {"dense": t}
        self._ws = {}
        self.whole_net = True   # run a LeNet-shaped graph as one kernel when no intermediate is wanted
        self._lenet = self._match_lenet()

    def _match_lenet(self):
        """The LeNet-shaped graph (Conv 5x5, Relu, MaxPool 2, Conv 5x5, Relu, MaxPool 2, Flatten, Gemm; 1 x 28 x 28
        input, 6 and 16 feature maps, binary weights) -> the three weight records, else None."""
        g = self.graph
        nodes = g["nodes"]
        ops = [n["op"] for n in nodes]
        if ops != ["Conv", "Relu", "MaxPool", "Conv", "Relu", "MaxPool", "Flatten", "Gemm"] or len(g["outputs"]) != 1:
            return None
        if any(nodes[i]["inputs"][0] != nodes[i - 1]["outputs"][0] for i in range(1, 8)):
            return None
        if nodes[7]["outputs"][0] not in g["outputs"] or len(g["inputs"]) != 1:
            return None
        shape = tuple(next(iter(g["inputs"].values())))
        if len(shape) != 4 or shape[1:] != (1, 28, 28):
            return None
        for c in (0, 3):
            a = nodes[c]["attrs"]
            if (list(a.get("strides", [1, 1])) != [1, 1] or any(a.get("pads", [0, 0, 0, 0])) or list(a.get("dilations", [1, 1])) != [1, 1]
                    or a.get("group", 1) != 1 or a.get("auto_pad", "NOTSET") not in ("NOTSET", "VALID")):
                return None
        for c in (2, 5):
            a = nodes[c]["attrs"]
            if (list(a.get("kernel_shape", [2, 2])) != [2, 2] or list(a.get("strides", a.get("kernel_shape", [2, 2]))) != [2, 2]
                    or any(a.get("pads", [0, 0, 0, 0])) or a.get("ceil_mode", 0)):
                return None
        a = nodes[7]["attrs"]
        if nodes[6]["attrs"].get("axis", 1) != 1 or a.get("transA", 0) or a.get("transB", 0) or a.get("alpha", 1.0) != 1.0 or a.get("beta", 1.0) != 1.0:
            return None
        recs = []
        for n, want in ((nodes[0], (6, 1, 5, 5)), (nodes[3], (16, 6, 5, 5)), (nodes[7], None)):
            w = self.weights.get(n["inputs"][1], {})
            if "words" not in w or (want is not None and (w["shape"] != want or w.get("order", 0) != capi.CONV_WEIGHTS_REFERENCE)):
                return None
            rec = {"words": w["words"], "alpha": w["alpha"]}
            if len(n["inputs"]) > 2:
                rec["bias"] = self.weights[n["inputs"][2]]["dense"]
            recs.append(rec)
        fshape = self.weights[nodes[7]["inputs"][1]]["shape"]
        if fshape[0] != 256 or not 1 <= fshape[1] <= 64:
            return None
        return recs + [fshape[1]]

    # -- weight preparation ----------------------------------------------------------------
    def _pack(self, w):
        L = self.L
        if w.dim() == 4:  # conv [M, C, kh, kw] -> K = C*kh*kw along the row: layout NK
            order = capi.CONV_WEIGHTS_TAP_MAJOR if (self.fast and w.shape[1] % 64 == 0) else capi.CONV_WEIGHTS_REFERENCE
            flat = L.permute_filters(w) if order else w.reshape(w.shape[0], -1)
            words_gt, alpha = L.quant_pack_binary(flat, capi.LAYOUT_NK, 0.0, False)
            # TBN mode uses the scale summed sequentially over the given weights, exactly as the reference
            # Session does (model.hpp:388-394); given a dequantised model (+-alpha weights) the whole Conv is
            # then bit-equal to the reference.
            alpha_seq = L.channel_abs_mean(flat.contiguous())
            return {"shape": tuple(w.shape), "words": words_gt, "alpha": alpha, "alpha_tbn": alpha_seq, "order": order}
        words_gt, alpha = L.quant_pack_binary(w, capi.LAYOUT_KN, 0.0, False)  # Gemm B [K, N]
        return {"shape": tuple(w.shape), "words": words_gt, "alpha": alpha}

    # -- reference surface -------------------------------------------------------------------
    def set_quantization(self, enable):
        self.quantization = bool(enable)

    def is_quantization_enabled(self):
        return self.quantization

    def set_input(self, name, array):
        if name not in self.graph["inputs"]:
            raise KeyError(f"Input '{name}' not found in model")
        t = array if self.torch.is_tensor(array) else self.torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32))
        if tuple(t.shape) != tuple(self.graph["inputs"][name]):
            raise ValueError(f"Input shape mismatch for '{name}'")
        self.inputs[name] = t.to(self.device, non_blocking=True)

    def get_output(self, name):
        if name not in self.values or name not in self.graph["outputs"]:
            raise KeyError(f"Output '{name}' not available")
        return self.values[name]

    def _workspace(self, key, nbytes):
        ws = self._ws.get(key)
        if ws is None or ws.numel() < nbytes:
            ws = self.torch.empty(max(nbytes, 256), dtype=self.torch.uint8, device=self.device)
            self._ws[key] = ws
        return ws

    # -- execution ---------------------------------------------------------------------------
    def run(self):
        if len(self.inputs) != len(self.graph["inputs"]):
            raise ValueError("Not all inputs provided")
        vals = dict(self.inputs)
        nodes = self.graph["nodes"]
        if (self._lenet is not None and self.whole_net and self.fuse and not self.quantization
                and not getattr(self, "keep_intermediates", True)):
            w1, w2, wf, classes = self._lenet
            out = self.L.lenet_fused(next(iter(self.inputs.values())), w1, w2, wf, classes)
            self.values = {nodes[-1]["outputs"][0]: out}
            self.intermediates = dict(self.values)
            return
        consumers = {}
        for n in nodes:
            for i in n["inputs"]:
                consumers[i] = consumers.get(i, 0) + 1
        # Index of the last node that reads each value: intermediates are released right after it, so a
        # large batch only ever holds the tensors that are still needed.
        last_use = {}
        for idx, n in enumerate(nodes):
            for i in n["inputs"]:
                last_use[i] = idx
        keep_all = getattr(self, "keep_intermediates", True)
        skip = set()
        self._cl = {}       # value name -> channels-last bf16 terms of that value (written by a chained convolution)
        self._shapes = {}   # value name -> NCHW shape, for values that exist only in the channels-last form
        self._chain_now = self.chain and not self.quantization
        self._readers = {}
        for n in nodes:
            for i in n["inputs"]:
                self._readers.setdefault(i, []).append(n)
        for idx, n in enumerate(nodes):
            if not keep_all:
                for name in [k for k, last in last_use.items() if last < idx and k in vals and k not in self.graph["outputs"]
                             and k not in self.inputs]:
                    del vals[name]
                    del last_use[name]
                    self._cl.pop(name, None)
            if idx in skip:
                continue
            op = n["op"]
            if op == "Conv":
                out_name, fused = self._conv(n, nodes, idx, vals, consumers, skip)
                vals[out_name] = fused
            elif op == "Gemm":
                vals[n["outputs"][0]] = self._gemm(n, vals)
            elif op == "Relu":
                vals[n["outputs"][0]] = self.L.relu(vals[n["inputs"][0]])
            elif op in ("MaxPool", "AveragePool"):
                a = n["attrs"]
                ks = a.get("kernel_shape", [2, 2])
                st = a.get("strides", ks)
                pd = a.get("pads", [0, 0, 0, 0])
                vals[n["outputs"][0]] = self.L.pool2d(0 if op == "MaxPool" else 1, vals[n["inputs"][0]],
                                                      (ks[0], ks[1], st[0], st[1], pd[0], pd[1]),
                                                      bool(a.get("ceil_mode", 0)), bool(a.get("count_include_pad", 0)))
            elif op == "GlobalAveragePool":
                vals[n["outputs"][0]] = self.L.global_avgpool2d(vals[n["inputs"][0]])
            elif op == "Flatten":
                x = vals[n["inputs"][0]]
                ax = n["attrs"].get("axis", 1)
                vals[n["outputs"][0]] = x.reshape(int(np.prod(x.shape[:ax])), -1)
            elif op == "Add":
                vals[n["outputs"][0]] = self.L.add(vals[n["inputs"][0]], vals[n["inputs"][1]])
            else:
                raise NotImplementedError(f"Operator '{op}' not implemented")
        self.values = {k: vals[k] for k in self.graph["outputs"]}
        self.intermediates = vals

    def _conv(self, n, nodes, idx, vals, consumers, skip):
        L = self.L
        a = n["attrs"]
        st = a.get("strides", [1, 1])
        pd = a.get("pads", [0, 0, 0, 0])
        dl = a.get("dilations", [1, 1])
        p = (st[0], st[1], pd[0], pd[1], dl[0], dl[1])  # only pads[0], pads[1] are honoured (model.hpp:313-321)
        in_name = n["inputs"][0]
        x = vals.get(in_name)          # None when the producer only wrote the channels-last form
        xshape = tuple(x.shape) if x is not None else self._shapes[in_name]
        w = self.weights[n["inputs"][1]]
        bias = self.weights[n["inputs"][2]]["dense"] if len(n["inputs"]) > 2 else None
        out_name = n["outputs"][0]
        order = w.get("order", capi.CONV_WEIGHTS_REFERENCE)
        ws = self._workspace("conv", L.h.tbn_conv2d_workspace_bytes(xshape[0], xshape[1], xshape[2], xshape[3],
                                                                    w["shape"][0], w["shape"][2], w["shape"][3], order))
        if self.quantization and "words" in w:
            y = L.conv2d_tbn(x, w["words"], w["shape"], p, alpha=w["alpha_tbn"], bias=bias,
                             epilogue=capi.EPI_BIAS_BEFORE_ALPHA, workspace=ws, order=order)
            return out_name, y
        # float x binary: fold a following Relu (and Add + Relu of a residual block) into the epilogue.
        epilogue, residual = 0, None
        # (a value that is also a graph output keeps its own name: nothing is folded over it)
        if self.fuse and consumers.get(out_name, 0) == 1 and out_name not in self.graph["outputs"] and idx + 1 < len(nodes):
            nxt = nodes[idx + 1]
            if nxt["op"] == "Relu" and nxt["inputs"] == [out_name]:
                epilogue |= capi.EPI_RELU
                skip.add(idx + 1)
                out_name = nxt["outputs"][0]
            elif (nxt["op"] == "Add" and out_name in nxt["inputs"] and idx + 2 < len(nodes)
                  and nodes[idx + 2]["op"] == "Relu" and nodes[idx + 2]["inputs"] == nxt["outputs"]
                  and consumers.get(nxt["outputs"][0], 0) == 1 and nxt["outputs"][0] not in self.graph["outputs"]):
                other = [i for i in nxt["inputs"] if i != out_name]
                if len(other) == 1 and vals.get(other[0]) is not None:
                    residual = vals[other[0]]
                    epilogue |= capi.EPI_RELU
                    skip.update((idx + 1, idx + 2))
                    out_name = nodes[idx + 2]["outputs"][0]
        if self._chain_now and order == capi.CONV_WEIGHTS_TAP_MAJOR:
            # Who reads the (possibly fused) result?  Channels-last convolutions take the bf16 form written by this
            # epilogue; anything else (a residual add, a pool, a graph output) needs the fp32 NCHW tensor.
            readers = self._readers.get(out_name, [])
            cl_readers = [r for r in readers if r["op"] == "Conv" and r["inputs"][0] == out_name
                          and self.weights[r["inputs"][1]].get("order") == capi.CONV_WEIGHTS_TAP_MAJOR]
            want_cl = len(cl_readers) > 0
            want_y = (len(cl_readers) != len(readers) or not readers or out_name in self.graph["outputs"]
                      or getattr(self, "keep_intermediates", True))
            x_cl = self._cl.get(in_name)
            y, y_cl = L.conv2d_chain(xshape, w, w["shape"], p, x=None if x_cl is not None else x, x_cl=x_cl, want_y=want_y,
                                     want_y_cl=want_cl, alpha=w.get("alpha"), bias=bias, residual=residual,
                                     epilogue=epilogue, workspace=ws, device=self.device)
            if y_cl is not None:
                self._cl[out_name] = y_cl
            self._shapes[out_name] = (xshape[0], w["shape"][0]) + tuple(
                L.conv_out_hw(xshape[2], xshape[3], w["shape"][2], w["shape"][3], p))
            return out_name, y
        if "words" in w:
            y = L.conv2d_fxb(x, w["words"], w["shape"], p, alpha=w["alpha"], bias=bias, residual=residual,
                             epilogue=epilogue, workspace=ws, order=order)
        else:
            y = L.conv2d_f32(x, w["split"], w["shape"], p, bias=bias, residual=residual, epilogue=epilogue, workspace=ws,
                             order=order)
        return out_name, y

    def _gemm(self, n, vals):
        L = self.L
        a = n["attrs"]
        if a.get("transA", 0) or a.get("transB", 0):
            raise NotImplementedError("transposed Gemm operands are not on the accelerated path yet")
        x = vals[n["inputs"][0]]
        w = self.weights[n["inputs"][1]]
        bias = self.weights[n["inputs"][2]]["dense"] if len(n["inputs"]) > 2 else None
        N = w["shape"][1]
        alpha_attr, beta = float(a.get("alpha", 1.0)), float(a.get("beta", 1.0))
        if bias is not None and beta != 1.0:
            bias = bias * beta
        if "words" not in w:
            ws = self._workspace("gemm", L.h.tbn_gemm_workspace_bytes(x.shape[0], x.shape[1], capi.MODE_TC_BF16X2))
            return L.gemm_f32(x.contiguous(), w["split"], N, alpha=alpha_attr, bias=bias, workspace=ws)
        if self.quantization:
            # Weights alpha*sign(w) are not exactly +-1, so the reference quantises them on the fly and runs
            # qlinear_matmul_binary with scale 1 (model.hpp:839-841), then alpha and beta*C (:845-869).
            ws = self._workspace("gemm", L.h.tbn_gemm_workspace_bytes(x.shape[0], x.shape[1], capi.MODE_TC_BF16X1))
            return L.gemm_tbn(x.contiguous(), w["words"], N, scale=alpha_attr, bias=bias, workspace=ws)
        ws = self._workspace("gemm", L.h.tbn_gemm_workspace_bytes(x.shape[0], x.shape[1], capi.MODE_TC_BF16X2))
        return L.gemm_fxb(x.contiguous(), w["words"], N, alpha=w["alpha"], scale=alpha_attr, bias=bias, workspace=ws)
