"""numpy front end of the CPU oracle (oracle/libgevva_golden.so). Test code only."""
import ctypes
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXPERTS, TOP_K, HIDDEN, INTER = 128, 8, 2816, 704


def _p(array):
    return array.ctypes.data_as(ctypes.c_void_p) if array is not None else None


def bf16_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def sf_bytes(routes, width):
    return (routes + EXPERTS * 127) * (width // 16)


class Oracle:
    def __init__(self):
        self.lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "libgevva_golden.so"))
        self.pin = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libgv_pin_toolkit.so"))
        ref = os.path.join(ROOT, "oracle", "_ref", "libgv_ref_decode.so")
        self.ref = ctypes.CDLL(ref) if os.path.exists(ref) else None
        L = self.lib
        f32, u8, u16, u32, i32 = (ctypes.c_float, ctypes.c_uint8, ctypes.c_uint16, ctypes.c_uint,
                                  ctypes.c_int)
        for name, args, res in (
                ("gvo_encode_e4m3", [f32], u8), ("gvo_decode_e4m3", [u8], f32),
                ("gvo_encode_e2m1", [f32], u8), ("gvo_decode_e2m1", [u32], f32),
                ("gvo_float_to_bf16", [f32], u16), ("gvo_bf16_to_float", [u16], f32),
                ("gvo_erff", [f32], f32), ("gvo_expf", [f32], f32), ("gvo_gelu", [f32], f32),
                ("gvo_sf_offset", [i32, i32, i32], ctypes.c_size_t), ("gvo_threads", [], i32)):
            getattr(L, name).argtypes = args
            getattr(L, name).restype = res
        L.gvo_pack_weight.restype = f32
        L.gvo_sort_routes.restype = i32
        L.gvo_moe_layer.restype = i32
        for name, res in (("pin_encode_e4m3", u8), ("pin_decode_e4m3", f32),
                          ("pin_encode_e2m1x2", u8), ("pin_float_to_bf16", u16)):
            getattr(self.pin, name).restype = res
        self.pin.pin_encode_e4m3.argtypes = [f32]
        self.pin.pin_decode_e4m3.argtypes = [u8]
        self.pin.pin_encode_e2m1x2.argtypes = [f32, f32]
        self.pin.pin_float_to_bf16.argtypes = [f32]
        if self.ref is not None:
            for name in ("ref_decode_e2m1", "ref_decode_e4m3"):
                getattr(self.ref, name).argtypes = [u32]
                getattr(self.ref, name).restype = f32

    # ---- stages ---------------------------------------------------------------
    def route(self, logits_bits, expert_scale_bits, act_scales=None, w_scale=None):
        tokens, ld = logits_bits.shape
        logits_bits = np.ascontiguousarray(logits_bits, dtype=np.uint16)
        weights = np.zeros((tokens, TOP_K), np.float32)
        ids = np.zeros((tokens, TOP_K), np.int32)
        self.lib.gvo_route(_p(logits_bits), ctypes.c_int(ld),
                           _p(np.ascontiguousarray(expert_scale_bits, dtype=np.uint16)),
                           _p(weights), _p(ids), ctypes.c_int(tokens), _p(act_scales), _p(w_scale))
        return weights, ids

    def router_logits(self, x, router, bias=None, e4m3=False):
        """x [tokens, 2816] and router [128, 2816] as bf16 bit patterns (uint16) or, with e4m3,
        as E4M3 bytes; returns bf16 logits [tokens, 128] as bit patterns."""
        tokens, width = x.shape
        logits = np.zeros((tokens, EXPERTS), np.uint16)
        bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self.lib.gvo_router_logits(_p(np.ascontiguousarray(x)), _p(np.ascontiguousarray(router)), _p(bias),
                                   ctypes.c_int(tokens), ctypes.c_int(width), ctypes.c_int(1 if e4m3 else 0),
                                   _p(logits))
        return logits

    def sort(self, ids):
        flat = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
        routes = flat.size
        out = {k: np.zeros(routes, np.int32) for k in ("sorted_experts", "sorted_routes", "inverse")}
        out["offsets"] = np.zeros(EXPERTS, np.int32)
        out["scale_rows"] = np.zeros(EXPERTS, np.int32)
        status = self.lib.gvo_sort_routes(_p(flat), ctypes.c_int(routes), _p(out["sorted_experts"]),
                                          _p(out["sorted_routes"]), _p(out["inverse"]),
                                          _p(out["offsets"]), _p(out["scale_rows"]))
        out["status"] = status
        return out

    def quantize_sorted(self, x_bits, in_scale_q, plan):
        tokens, width = x_bits.shape
        routes = tokens * TOP_K
        packed = np.zeros((routes, width // 2), np.uint8)
        scales = np.zeros(sf_bytes(routes, width), np.uint8)
        self.lib.gvo_quantize_sorted(_p(np.ascontiguousarray(x_bits)), _p(in_scale_q),
                                     _p(plan["sorted_experts"]), _p(plan["sorted_routes"]),
                                     _p(plan["offsets"]), _p(plan["scale_rows"]),
                                     ctypes.c_int(width), ctypes.c_int(routes), _p(packed), _p(scales))
        return packed, scales

    def geglu_quantize(self, fused_bits, in_scale_q, plan):
        routes = fused_bits.shape[0]
        packed = np.zeros((routes, INTER // 2), np.uint8)
        scales = np.zeros(sf_bytes(routes, INTER), np.uint8)
        self.lib.gvo_geglu_quantize(_p(np.ascontiguousarray(fused_bits)), _p(in_scale_q),
                                    _p(plan["sorted_experts"]), _p(plan["offsets"]),
                                    _p(plan["scale_rows"]), ctypes.c_int(routes), _p(packed),
                                    _p(scales))
        return packed, scales

    def grouped_gemm(self, a_packed, a_scales, plan, w, w_sf, alpha, n_out, k_in):
        routes = a_packed.shape[0]
        out = np.zeros((routes, n_out), np.uint16)
        self.lib.gvo_grouped_gemm(_p(a_packed), _p(a_scales), _p(plan["offsets"]),
                                  _p(plan["scale_rows"]), ctypes.c_int(routes), _p(w), _p(w_sf),
                                  _p(alpha), ctypes.c_int(n_out), ctypes.c_int(k_in), _p(out))
        return out

    def reduce(self, routed_bits, route_weights, inverse, tokens):
        out = np.zeros((tokens, HIDDEN), np.uint16)
        self.lib.gvo_reduce_routes(_p(np.ascontiguousarray(routed_bits)),
                                   _p(np.ascontiguousarray(route_weights, dtype=np.float32)),
                                   _p(inverse), ctypes.c_int(tokens), _p(out))
        return out

    def pack_weight(self, w):
        n_out, k_in = w.shape
        w = np.ascontiguousarray(w, dtype=np.float32)
        codes = np.zeros((n_out, k_in // 2), np.uint8)
        scales = np.zeros((n_out, k_in // 16), np.uint8)
        g = self.lib.gvo_pack_weight(_p(w), ctypes.c_int(n_out), ctypes.c_int(k_in), _p(codes),
                                     _p(scales))
        return codes, scales, np.float32(g)

    def moe_layer(self, x_bits, ids, route_weights, weights, want_routed=False):
        """weights: dict of numpy arrays w13,w13_sf,w2,w2_sf,alpha1,alpha2,in_scale_q1,in_scale_q2."""
        tokens = x_bits.shape[0]
        out = np.zeros((tokens, HIDDEN), np.uint16)
        routed = np.zeros((tokens * TOP_K, HIDDEN), np.uint16) if want_routed else None
        inverse = np.zeros(tokens * TOP_K, np.int32) if want_routed else None
        status = self.lib.gvo_moe_layer(
            _p(np.ascontiguousarray(x_bits)), _p(np.ascontiguousarray(ids, dtype=np.int32)),
            _p(np.ascontiguousarray(route_weights, dtype=np.float32)), ctypes.c_int(tokens),
            _p(weights["w13"]), _p(weights["w13_sf"]), _p(weights["w2"]), _p(weights["w2_sf"]),
            _p(weights["alpha1"]), _p(weights["alpha2"]), _p(weights["in_scale_q1"]),
            _p(weights["in_scale_q2"]), _p(out), _p(routed), _p(inverse))
        assert status == 0
        return (out, routed, inverse) if want_routed else out


class DenseOracle:
    """Dense FP8 MLP and feed-forward pre/post steps of the oracle."""

    def __init__(self, oracle):
        self.lib = oracle.lib
        self.lib.gvo_pack_fp8_weight.restype = ctypes.c_float

    def ff_prepare(self, x, dense_w, expert_w, router_scale):
        rows = x.shape[0]
        outs = [np.zeros((rows, HIDDEN), np.uint16) for _ in range(3)]
        self.lib.gvo_ff_prepare(_p(np.ascontiguousarray(x)), _p(dense_w), _p(expert_w), _p(router_scale),
                                _p(outs[0]), _p(outs[1]), _p(outs[2]), ctypes.c_int(rows))
        return outs

    def quantize_rows(self, x):
        rows, width = x.shape
        out = np.zeros((rows, width), np.uint8)
        scales = np.zeros(rows, np.float32)
        self.lib.gvo_fp8_quantize_rows(_p(np.ascontiguousarray(x)), ctypes.c_int(rows), ctypes.c_int(width),
                                       _p(out), _p(scales))
        return out, scales

    def gemm(self, a, w):
        rows, k = a.shape
        n = w.shape[0]
        out = np.zeros((rows, n), np.uint16)
        self.lib.gvo_fp8_gemm_unscaled(_p(np.ascontiguousarray(a)), _p(np.ascontiguousarray(w)),
                                       ctypes.c_int(rows), ctypes.c_int(n), ctypes.c_int(k), _p(out))
        return out

    def gelu_quantize(self, gate_up, act_scales, gate_scale, up_scale):
        rows = gate_up.shape[0]
        out = np.zeros((rows, 2112), np.uint8)
        scales = np.zeros(rows, np.float32)
        self.lib.gvo_gelu_quantize_fp8(_p(np.ascontiguousarray(gate_up)), _p(act_scales),
                                       ctypes.c_float(gate_scale), ctypes.c_float(up_scale),
                                       ctypes.c_int(rows), _p(out), _p(scales))
        return out, scales

    def finalize(self, dense, dense_w, routes, route_weights, inverse, expert_w, combined_w, residual,
                 layer_scalar_bits, act_scales, proj_scale):
        rows = dense.shape[0]
        out = np.zeros((rows, HIDDEN), np.uint16)
        self.lib.gvo_ff_finalize(_p(np.ascontiguousarray(dense)), _p(dense_w), _p(np.ascontiguousarray(routes)),
                                 _p(np.ascontiguousarray(route_weights, dtype=np.float32)), _p(inverse),
                                 _p(expert_w), _p(combined_w), _p(np.ascontiguousarray(residual)),
                                 ctypes.c_uint16(int(layer_scalar_bits)), _p(out), ctypes.c_int(rows),
                                 _p(act_scales), ctypes.c_float(proj_scale))
        return out

    def pack_fp8(self, w):
        w = np.ascontiguousarray(w, dtype=np.float32)
        out = np.zeros(w.shape, np.uint8)
        scale = self.lib.gvo_pack_fp8_weight(_p(w), ctypes.c_size_t(w.size), _p(out))
        return out, np.float32(scale)
