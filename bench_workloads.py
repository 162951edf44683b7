"""Layer tables of the benchmark configurations (shapes only: no arithmetic).

Each table is a list of dicts in network order with the geometry the factor
kernels need; ``layer_dims`` gives (dA, dG, rows_A, rows_G) of a layer, where a
factor side includes the bias column when the layer has a bias.  Used by
``bench.py`` and by the full-shape parity tests.
"""


def conv_out_size(size, k, s, p):
    return (size + 2 * p - k) // s + 1


def _conv(layers, name, cin, cout, k, s, p, hin, batch, bias=False):
    ho = conv_out_size(hin, k, s, p)
    layers.append(dict(name=name, kind='conv', cin=cin, cout=cout, k=k,
                       stride=s, pad=p, hin=hin, hout=ho, bias=bias, n=batch))
    return ho


def resnet50_layers(batch=32, image=224, classes=1000):
    """Vanilla ResNet-50 (v1.5: stride on the 3x3): 53 convolutions + 1 fully
    connected layer; only conv1 and fc carry a bias."""
    layers = []
    h = _conv(layers, 'conv1', 3, 64, 7, 2, 3, image, batch, bias=True)
    h = conv_out_size(h, 3, 2, 1)  # 3x3/2 max pool
    cin = 64
    for stage, (blocks, mid) in enumerate(
            [(3, 64), (4, 128), (6, 256), (3, 512)], start=1):
        for b in range(blocks):
            s = 2 if (b == 0 and stage > 1) else 1
            pre = 'res%d.%d.' % (stage, b)
            hin = h
            _conv(layers, pre + 'conv1', cin, mid, 1, 1, 0, hin, batch)
            h2 = _conv(layers, pre + 'conv2', mid, mid, 3, s, 1, hin, batch)
            _conv(layers, pre + 'conv3', mid, mid * 4, 1, 1, 0, h2, batch)
            if b == 0:
                _conv(layers, pre + 'short', cin, mid * 4, 1, s, 0, hin, batch)
            cin = mid * 4
            h = h2
    layers.append(dict(name='fc', kind='linear', cin=cin, cout=classes,
                       bias=True, n=batch))
    return layers


def bn_layers_of(layers):
    """The BatchNormalization layers of a network whose every convolution is
    followed by one (ResNet-50: 53, CIFAR ResNet-18: 20): channels and
    spatial size of the convolution's output."""
    return [dict(name=l['name'] + '.bn', kind='bn', c=l['cout'], h=l['hout'],
                 n=l['n'], bias=True) for l in layers if l['kind'] == 'conv']


def resnet18_cifar_layers(batch=128, image=32, classes=10):
    """CIFAR-style ResNet-18: 3x3 stem, four stages of two basic blocks
    (64/128/256/512 channels), 1x1 shortcuts where the shape changes, fc
    512 -> classes with bias.  20 convolutions + 1 fully connected layer."""
    layers = []
    h = _conv(layers, 'conv1', 3, 64, 3, 1, 1, image, batch)
    cin = 64
    for stage, cout in enumerate([64, 128, 256, 512], start=1):
        for b in range(2):
            s = 2 if (b == 0 and stage > 1) else 1
            pre = 'res%d.%d.' % (stage, b)
            hin = h
            h = _conv(layers, pre + 'conv1', cin, cout, 3, s, 1, hin, batch)
            _conv(layers, pre + 'conv2', cout, cout, 3, 1, 1, h, batch)
            if s != 1 or cin != cout:
                _conv(layers, pre + 'short', cin, cout, 1, s, 0, hin, batch)
            cin = cout
    layers.append(dict(name='fc', kind='linear', cin=cin, cout=classes,
                       bias=True, n=batch))
    return layers


def mlp_layers(batch=128, sizes=(784, 1000, 1000, 10)):
    """MNIST-shaped multi-layer perceptron, every layer with a bias."""
    return [dict(name='l%d' % (i + 1), kind='linear', cin=a, cout=b, bias=True,
                 n=batch) for i, (a, b) in enumerate(zip(sizes, sizes[1:]))]


def block_factors(layer):
    """[(side, rows of the matrix it is built from), ...] for the factors of a
    layer's curvature block: (A, G) of a connection, F of side 2c built from
    the n per-sample gradients for BatchNormalization."""
    if layer['kind'] == 'bn':
        return [(2 * layer['c'], layer['n'])]
    dA, dG, rA, rG = layer_dims(layer)
    return [(dA, rA), (dG, rG)]


def layer_dims(layer):
    """(dA, dG, rows_A, rows_G) of a connection layer dict; for a
    BatchNormalization layer (2c, 0, n, 0)."""
    if layer['kind'] == 'bn':
        return 2 * layer['c'], 0, layer['n'], 0
    if layer['kind'] == 'linear':
        return (layer['cin'] + int(layer['bias']), layer['cout'],
                layer['n'], layer['n'])
    dA = layer['cin'] * layer['k'] ** 2 + int(layer['bias'])
    rows = layer['n'] * layer['hout'] ** 2
    return dA, layer['cout'], rows, rows


def distinct_shapes(layers):
    """One layer per distinct geometry, with its multiplicity."""
    groups = {}
    for l in layers:
        key = (l['kind'], l.get('k'), l.get('stride'), l.get('pad'),
               l.get('cin'), l.get('cout'), l.get('hin'), l.get('c'),
               l.get('h'), l['bias'], l['n'])
        groups.setdefault(key, [l, 0])[1] += 1
    return [(l, m) for l, m in groups.values()]
