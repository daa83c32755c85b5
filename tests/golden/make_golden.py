"""Collects the golden-vector models the reference ships for the quantized operator path.

Run in a container that has the reference checkout:  python tests/golden/make_golden.py /path/to/reference
It copies the small `.espdl` test models that embed `test_inputs_value` / `test_outputs_value`
(the data the reference's own `Model::test()` checks, test_apps/esp-dl/main/test_dl_model.cpp:14-52)
into tests/golden/espdl/<target>__<name>.espdl, byte for byte.  They are data files, a few KB each.

It also copies two of the model-zoo files (models/imagenet_cls, models/coco_detect; 3-4 MB each, ESP32-P4 filter layout,
per-channel exponents, no embedded test vectors): the ImageNet MobileNetV2 classifier and the YOLO11n detector at 320x320.
The tests run them on seeded random images and compare the backend with the graph oracle.
"""
import os
import shutil
import sys

if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py /path/to/reference-checkout")
REF = sys.argv[1]
HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "espdl")

SOURCES = []
for target in ("c", "esp32p4", "esp32s3"):
    d = os.path.join(REF, "test_apps/esp-dl/models", target, "Gemm")
    for f in sorted(os.listdir(d)):
        if f.endswith(".espdl"):
            SOURCES.append((os.path.join(d, f), f"{target}__{f}"))
for chip, target in (("p4", "esp32p4"), ("s3", "esp32s3")):
    SOURCES.append((os.path.join(REF, "examples/tutorial/how_to_run_model/main/models", chip, "model.espdl"),
                    f"{target}__sin_mlp.espdl"))
for target in ("esp32p4", "esp32s3"):
    SOURCES.append((os.path.join(REF, "examples/tutorial/how_to_deploy_streaming_model/test_streaming_model/main/models",
                                 target, "model.espdl"), f"{target}__streaming_tcn.espdl"))
    SOURCES.append((os.path.join(REF, "examples/tutorial/how_to_deploy_streaming_model/test_streaming_model/main/models",
                                 target, "streaming_model.espdl"), f"{target}__streaming_tcn_chunked.espdl"))

SOURCES.append((os.path.join(REF, "models/imagenet_cls/models/p4/imagenet_cls_mobilenetv2_s8_v1.espdl"), "esp32p4__zoo_mobilenetv2.espdl"))
SOURCES.append((os.path.join(REF, "models/coco_detect/models/p4/coco_detect_yolo11n_320_s8_v1.espdl"), "esp32p4__zoo_yolo11n_320.espdl"))

# smaller model-zoo files that bring operators and layouts the two above do not have: an ESP32-S3 layout (half-up rounding),
# PRelu with per-channel slopes, InsertZeros (transposed-convolution halves) with rectangular pool strides, and the
# detector / re-identification topologies
for src, name in (("models/human_face_detect/models/p4/human_face_detect_msr_s8_v1.espdl", "esp32p4__zoo_face_msr.espdl"),
                  ("models/human_face_detect/models/s3/human_face_detect_msr_s8_v1.espdl", "esp32s3__zoo_face_msr.espdl"),
                  ("models/human_face_detect/models/p4/human_face_detect_mnp_s8_v1.espdl", "esp32p4__zoo_face_mnp.espdl"),
                  ("models/pedestrian_detect/models/p4/pedestrian_detect_pico_s8_v1.espdl", "esp32p4__zoo_pedestrian_pico.espdl"),
                  ("models/person_reid/models/p4/person_reid_feat_osn_s8_v1.espdl", "esp32p4__zoo_person_reid.espdl"),
                  ("models/pp_ocr_v6/models/p4/pp_ocr_v6_det_s8.espdl", "esp32p4__zoo_ocr_det.espdl")):
    SOURCES.append((os.path.join(REF, src), name))



def write_topology(src, dst):
    """Writes the graph of a model file WITHOUT its weights as JSON: nodes with their attributes, every tensor's
    shape, element type and exponent, and for each parameter its dims, element type and number of exponents.  Values
    are kept only for the small constants that are part of the graph's structure (Reshape / Split / Slice / Resize
    operands, the scalar of a Mul): at most 16 elements, and never a Conv operand or a table.  The 640x640 YOLO11n
    file is used this way: its topology at full size is needed (249 nodes), its 2.6 MB of trained weights are not -
    `espdl_b200.zoo.from_topology` fills the graph with seeded random weights."""
    import json
    sys.path.insert(0, os.path.join(HERE, "..", ".."))
    import __graft_entry__ as entry
    entry._package()
    from espdl_b200 import espdl_file
    m = espdl_file.read(src)
    weights = set()
    for n in m["nodes"]:
        if n["op_type"] in ("Conv", "Gemm"):
            weights.update(n["inputs"][1:])
        if "lut" in n["attrs"] and isinstance(n["attrs"]["lut"], str):
            weights.add(n["attrs"]["lut"])
    def vinfo(v):
        return dict(name=v["name"], elem_type=v["elem_type"], shape=v["shape"], exponents=v["exponents"])
    params = {}
    for name, t in m["initializers"].items():
        entry_ = dict(dims=t["dims"], data_type=t["data_type"], n_exponents=len(t["exponents"]))
        if name not in weights and t["data"] is not None and t["data"].size <= 16:
            entry_["values"] = [float(x) if t["data"].dtype.kind == "f" else int(x) for x in t["data"].reshape(-1)]
            entry_["exponents"] = t["exponents"]
        params[name] = entry_
    topo = dict(source=os.path.relpath(src, REF), nodes=[dict(op_type=n["op_type"], name=n["name"], inputs=n["inputs"], outputs=n["outputs"],
                                                                attrs={k: v for k, v in n["attrs"].items() if not isinstance(v, dict)})
                                                           for n in m["nodes"]],
                inputs=[vinfo(v) for v in m["inputs"]], outputs=[vinfo(v) for v in m["outputs"]],
                value_info=[vinfo(v) for v in m["value_info"].values()], parameters=params)
    with open(dst, "w") as f:
        json.dump(topo, f, separators=(",", ":"))
    print(f"{os.path.basename(dst)}: {len(topo['nodes'])} nodes, {os.path.getsize(dst)} bytes")


if __name__ == "__main__":
    os.makedirs(OUT, exist_ok=True)
    for src, name in SOURCES:
        shutil.copyfile(src, os.path.join(OUT, name))
        print(f"{name}: {os.path.getsize(src)} bytes")
    write_topology(os.path.join(REF, "models/coco_detect/models/p4/coco_detect_yolo11n_s8_v1.espdl"), os.path.join(HERE, "yolo11n_640_topology.json"))
