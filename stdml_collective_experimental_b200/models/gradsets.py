"""Gradient-set shapes of the benchmark models, generated from the model
architectures (not copied from the reference's testdata files).

The reference benchmarks all-reduce over files of tensor sizes
(testdata/resnet50.txt = 214 entries incl. BN running statistics, vgg16.txt =
32, bert.txt = 599 = BERT-base weights plus two optimizer slots).  Here the
sets are the TRAINABLE tensors only: ResNet-50 161 tensors / 25,557,032
elements, VGG16 32 / 138,357,544, BERT-base 199 / ~109.5 M, BERT-large
391 / ~335 M.  Two more sets restate what the reference's own files describe,
for like-for-like runs against its binaries: `resnet50-214` (the 53
convolutions carry a bias: 214 tensors / 25,583,592 elements) and `bert-599`
(BERT-base with its pooler and a 2-way classifier, 201 tensors, followed by two
optimizer slots for each of the 199 tensors below the pooler: 599 tensors /
327,270,150 elements).  `SWEEP` is the reference's `AxB` list
(testdata/test-set-1.txt).
"""
from functools import reduce
from operator import mul


def _numel(shape):
    return reduce(mul, shape, 1)


def resnet50_shapes(num_classes=1000):
    shapes = [(64, 3, 7, 7), (64,), (64,)]
    inplanes = 64
    for planes, blocks in ((64, 3), (128, 4), (256, 6), (512, 3)):
        for b in range(blocks):
            shapes += [(planes, inplanes, 1, 1), (planes,), (planes,),
                       (planes, planes, 3, 3), (planes,), (planes,),
                       (planes * 4, planes, 1, 1), (planes * 4,), (planes * 4,)]
            if b == 0:
                shapes += [(planes * 4, inplanes, 1, 1), (planes * 4,), (planes * 4,)]
            inplanes = planes * 4
    shapes += [(num_classes, 2048), (num_classes,)]
    return shapes


def vgg16_shapes(num_classes=1000):
    cfg = [64, 64, 128, 128, 256, 256, 256, 512, 512, 512, 512, 512, 512]
    shapes, cin = [], 3
    for cout in cfg:
        shapes += [(cout, cin, 3, 3), (cout,)]
        cin = cout
    shapes += [(4096, 512 * 7 * 7), (4096,), (4096, 4096), (4096,), (num_classes, 4096),
               (num_classes,)]
    return shapes


def bert_shapes(layers, hidden, ffn, vocab=30522, max_pos=512, type_vocab=2):
    shapes = [(vocab, hidden), (max_pos, hidden), (type_vocab, hidden), (hidden,), (hidden,)]
    for _ in range(layers):
        for _ in range(4):  # q, k, v, attention output
            shapes += [(hidden, hidden), (hidden,)]
        shapes += [(hidden,), (hidden,)]  # attention LayerNorm
        shapes += [(ffn, hidden), (ffn,), (hidden, ffn), (hidden,)]
        shapes += [(hidden,), (hidden,)]  # output LayerNorm
    shapes += [(hidden, hidden), (hidden,)]  # pooler
    return shapes


def bert_base_shapes():
    return bert_shapes(12, 768, 3072)


def bert_large_shapes():
    return bert_shapes(24, 1024, 4096)


def resnet50_with_conv_bias_shapes(num_classes=1000):
    shapes = []
    for sh in resnet50_shapes(num_classes):
        shapes.append(sh)
        if len(sh) == 4:
            shapes.append((sh[0],))
    return shapes


def bert_finetune_with_slots_shapes():
    body = bert_shapes(12, 768, 3072)[:-2]  # everything below the pooler
    head = [(2, 768), (2,)]
    weights = body + [(768, 768), (768,)] + head
    slots = []
    for sh in body + head:
        slots += [sh, sh]  # first and second moment, side by side
    return weights + slots


SWEEP = ["1024x100", "2048x100", "4096x100", "8192x100", "16384x100", "102400x100",
         "1024000x100", "10240000x10", "262144x10"]

GRADSETS = {
    "resnet50-214": resnet50_with_conv_bias_shapes,
    "bert-599": bert_finetune_with_slots_shapes,
    "resnet50": resnet50_shapes,
    "vgg16": vgg16_shapes,
    "bert-base": bert_base_shapes,
    "bert-large": bert_large_shapes,
}


def gradset_sizes(name):
    """Element counts of the named gradient set, or of an `AxB` workload
    (B tensors of A elements, the reference benchmarks' syntax)."""
    if name in GRADSETS:
        return [_numel(s) for s in GRADSETS[name]()]
    if "x" in name:
        a, b = name.split("x")
        return [int(a)] * int(b)
    raise KeyError(f"unknown gradient set {name!r}")


def write_sizes_file(name, path):
    """One element count per line: the input format of the reference's
    bench-all-reduce and of this package's C++ benchmarks."""
    with open(path, "w") as f:
        for n in gradset_sizes(name):
            f.write(f"{n}\n")
    return path
