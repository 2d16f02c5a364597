"""Python interface of the CUDA (sm_100a) deepRacin library.

Mirrors the reference's ctypes module (python/deepracin/__init__.py.in): the same
``Environment`` / ``Graph`` / ``Node`` objects, the same free functions (``feed_node``,
``prepare``, ``apply``, ``feed_data``, ``mark_as_output``, ``load_graph``, ``save_graph``,
``Conv2d``, ``Fully_Connected``, ``Pooling``, ``Softmax``, ``Slice``, ``Concat``,
``Crop_Or_Pad``, the scalar and element-wise ops) with the same argument meaning and the
same layout handling: the user speaks ``HWC`` (default), ``CHW`` or ``WHC``; the C API is
fed [C][H][W] buffers and weights are transposed HWIO -> [Cin][Cout][kh][kw]
(__init__.py.in:458-462, 487-489, 559-562).

Additions: ``Graph.batch`` (images per ``apply``; arrays gain a leading batch axis),
``Graph.math`` ('fp32' | 'tf32' | 'fp32x3'), ``Graph.conv_algo``, ``Graph.autotune``, ``Graph.cuda_graph``,
``Graph.feed_overlap``.

All computation happens in ``libdeepracin.so`` on the GPU; there is no CPU path here.
"""
import ctypes
import os
import shutil
import tempfile
from ctypes import POINTER, byref, c_float, c_int, c_void_p, pointer

import numpy as np

from ._lib import Shape2, Shape3, Shape4, load

lib = load()

act_dict = {"linear": 0, "relu": 1}
pool_dict = {"max": 0, "average": 1}
MATH = {"fp32": 0, "tf32": 1, "fp32x3": 2}
CONV_ALGO = {"auto": 0, "direct": 1, "winograd": 2, "1x1": 3, "tensor": 4, "tensor_winograd": 5, "winograd4": 6}
_FP = POINTER(c_float)


def _fptr(a):
    return None if a is None else a.ctypes.data_as(_FP)


class Node:
    def __init__(self, ptr, graph, desc, params, variables=None):
        if not ptr:
            raise RuntimeError("DR Error: node '%s' could not be created" % desc)
        self.ptr = ptr
        self.graph = graph
        self.desc = desc
        self.params = params
        self.variables = variables
        self.out_shape = None
        self.shape = None
        graph.nodes.append(self)

    def __add__(self, other):
        return Add(self, other) if isinstance(other, Node) else Add_Scalar(self, other)

    def __sub__(self, other):
        return Sub(self, other) if isinstance(other, Node) else Sub_Scalar(self, other)

    def __mul__(self, other):
        return Mul(self, other) if isinstance(other, Node) else Mul_Scalar(self, other)

    def __truediv__(self, other):
        return Div(self, other) if isinstance(other, Node) else Div_Scalar(self, other)

    def __pow__(self, power, modulo=None):
        return Pow(self, power) if isinstance(power, Node) else Pow_Scalar(self, power)


class Graph:
    def __init__(self, id, layout, env):
        self.ptr = lib.dR_NewGraph()
        self.num_outputs = 0
        self.outnodes = []
        self.id = id
        self.layout = layout
        self.nodes = []
        self.feed_nodes = []
        self.model_path = None
        self.env = env
        self.batch = 1
        self.math = "fp32"
        self.conv_algo = "auto"
        self.autotune = False
        self.fuse = True
        self.cuda_graph = False
        self.feed_overlap = False
        self.prepared = False

    def gpu_ms(self, iterations=1):
        """dR_apply timed with events on the graph's own stream (ms for `iterations` applies)."""
        return lib.dR_applyTimed(self.ptr, iterations)


class Environment:
    def __init__(self, preferred_platform="", device=0):
        self.preferred_platform_name = preferred_platform
        self.device = device

    def __enter__(self):
        self.silent = True
        self.debuginfo = False
        self.profileCPU = False
        self.profileGPU = False
        self.tmp_path = tempfile.mkdtemp(prefix="deepracin_")
        self.model_path = self.tmp_path
        self.graphs = []
        self.graph_with_cl_context = -1
        self.id_counter = 0
        return self

    def __exit__(self, type, value, traceback):
        shutil.rmtree(self.tmp_path, ignore_errors=True)
        # graphs that borrowed the environment's stream go first; the graph that created it tears it down last
        owner = self.graph_with_cl_context
        for graph in self.graphs:
            if graph.id != owner:
                lib.dR_cleanup(graph.ptr, 0)
        for graph in self.graphs:
            if graph.id == owner:
                lib.dR_cleanup(graph.ptr, 1)
        self.graphs = []

    def create_graph(self, interface_layout="HWC"):
        if interface_layout not in ("HWC", "CHW", "WHC"):
            raise NotImplementedError("DR Error: Graphs's layout " + interface_layout + " not supported!")
        graph = Graph(self.id_counter, interface_layout, self)
        self.id_counter += 1
        self.graphs.append(graph)
        return graph


def _to_dr_shape3(layout, shape):
    """user (layout-ordered) 3-shape -> deepRacin (W, H, C)"""
    if layout == "WHC":
        return [shape[0], shape[1], shape[2]]
    if layout == "CHW":
        return [shape[2], shape[1], shape[0]]
    return [shape[1], shape[0], shape[2]]


def feed_node(graph, shape):
    if len(shape) != 3 or not all(isinstance(s, (int, np.integer)) for s in shape):
        raise TypeError("DR Error: feed_node()'s shape parameter needs to be a list with 3 ints!")
    d = _to_dr_shape3(graph.layout, [int(s) for s in shape])
    sh = Shape3(*d)
    node = Node(lib.dR_Datafeednode(graph.ptr, pointer(sh)), graph, "DataFeedNode", d)
    graph.feed_nodes.append(node)
    return node


def prepare(graph):
    env = graph.env
    lib.dR_setBatchSize(graph.ptr, int(graph.batch))
    lib.dR_setMathMode(graph.ptr, MATH[graph.math])
    lib.dR_setGraphConvAlgo(graph.ptr, CONV_ALGO[graph.conv_algo])
    lib.dR_setAutotune(graph.ptr, 1 if graph.autotune else 0)
    lib.dR_setFusion(graph.ptr, 1 if graph.fuse else 0)
    lib.dR_setCudaGraph(graph.ptr, 1 if graph.cuda_graph else 0)
    lib.dR_setFeedOverlap(graph.ptr, 1 if graph.feed_overlap else 0)
    if env.graph_with_cl_context == -1:
        model_path = graph.model_path if graph.model_path is not None else env.model_path
        os.makedirs(model_path, exist_ok=True)
        lib.dR_config(graph.ptr, env.preferred_platform_name.encode(), env.silent, env.debuginfo, env.profileGPU, env.profileCPU,
                      model_path.encode())
        lib.dR_setDevice(graph.ptr, int(env.device))
        if not lib.dR_initCL(graph.ptr):
            raise RuntimeError("DR Error: deepRACIN initCL failed!")
        env.graph_with_cl_context = graph.id
    else:
        lib.dR_getClEnvironmentFrom(graph.ptr, env.graphs[env.graph_with_cl_context].ptr)
    if not lib.dR_prepare(graph.ptr):
        raise RuntimeError("DR Error: deepRACIN prepare failed!")
    for node in graph.outnodes:
        s = lib.dR_getOutputShape(node.ptr).contents
        node.out_shape = [s.s0, s.s1, s.s2]
    for feednode in graph.feed_nodes:
        s = lib.dR_getOutputShape(feednode.ptr).contents
        feednode.shape = [s.s0, s.s1, s.s2]
    graph.prepared = True


def _from_chw(layout, arr):
    """[n, C, H, W] -> user layout (keeps the batch axis first)"""
    if layout == "WHC":
        return arr.transpose([0, 3, 2, 1])
    if layout == "HWC":
        return arr.transpose([0, 2, 3, 1])
    return arr


def fetch(graph):
    """Downloads every output (blocking); arrays in the graph's layout, batch axis first when batch > 1."""
    memptr = (c_void_p * max(graph.num_outputs, 1))()
    lib.dR_getOutputBuffers(graph.ptr, memptr)
    out = []
    for i in range(graph.num_outputs):
        w, h, c = graph.outnodes[i].out_shape
        arr = np.empty((graph.batch, c, h, w), np.float32)
        lib.dR_downloadArray(graph.ptr, b"output", memptr[i], 0, arr.nbytes, arr.ctypes.data_as(c_void_p))
        arr = _from_chw(graph.layout, arr)
        out.append(np.squeeze(arr) if graph.batch == 1 else arr)
    return out


def apply(graph):
    if not lib.dR_apply(graph.ptr):
        raise RuntimeError("DR Error: deepRACIN apply failed!")
    return fetch(graph)


def mark_as_output(node):
    lib.dR_setAsOutput(node.graph.ptr, node.ptr)
    node.graph.num_outputs += 1
    node.graph.outnodes.append(node)


def feed_data(node, data):
    graph = node.graph
    data = np.asarray(data)
    if data.dtype != np.float32:
        raise TypeError("DR Error: data fed to a feed_node is " + str(data.dtype) + " but needs to be an array of type float32!")
    if data.ndim == 3:
        data = data[None]
    if data.ndim != 4 or data.shape[0] != graph.batch:
        raise TypeError("DR Error: data fed to a feed_node needs 3 dimensions (or 4 with a leading batch axis of %d)!" % graph.batch)
    if graph.layout == "WHC":
        chw = data.transpose([0, 3, 2, 1])
    elif graph.layout == "HWC":
        chw = data.transpose([0, 3, 1, 2])
    else:
        chw = data
    dr_shape = [chw.shape[3], chw.shape[2], chw.shape[1]]
    if dr_shape != node.shape:
        raise ValueError("DR Error: data array's dimensions " + str(dr_shape) + " do not match node's dimensions " + str(node.shape) + "!")
    chw = np.ascontiguousarray(chw)
    lib.dR_feedData(graph.ptr, node.ptr, _fptr(chw), 0, chw.size)


def load_graph(graph, path):
    if not isinstance(path, str):
        raise TypeError("DR Error: Load graph needs graph folder path!")
    graph.model_path = path
    num_nodes, num_feed = c_int(0), c_int(0)
    nodesptr, feedptr = POINTER(c_void_p)(), POINTER(c_void_p)()
    last = lib.dR_loadGraph(graph.ptr, path.encode(), byref(nodesptr), byref(num_nodes), byref(feedptr), byref(num_feed))
    if not last:
        raise RuntimeError("DR Error: Model could not be loaded!")
    nodelist = [Node(nodesptr[i], graph, None, None) for i in range(num_nodes.value)]
    feednodelist = [Node(feedptr[i], graph, None, None) for i in range(num_feed.value)]
    graph.feed_nodes = feednodelist
    return nodelist, feednodelist


def save_graph(graph, path):
    if not lib.dR_saveGraph(graph.ptr, path.encode()):
        raise RuntimeError("DR Error: Model could not be saved!")


def print_graph(graph):
    lib.dR_printNetObject(graph.ptr, None)


# ------------------------------------------------------------------------------- layers
def Conv2d(input_node, shape, stride, activation, weights, biases=None, algo=None):
    """shape = (kh, kw, Cin, Cout) with kh == kw, stride = (1, s, s, 1); weights HWIO."""
    if not shape[0] == shape[1]:
        raise TypeError("DR Error: Conv2d' currently only supports quadratic filter sizes!")
    if not (stride[0] == stride[3] == 1):
        raise TypeError("DR Error: Conv2d' currently only strides of from (1,x,y,1)!")
    if activation not in act_dict:
        raise ValueError("DR Error: Activation parameter needs to be 'relu' or 'linear'!")
    use_bias = biases is not None
    w = None
    if weights is not None:
        w = np.ascontiguousarray(np.asarray(weights, np.float32).transpose([2, 3, 0, 1]))
    b = None if biases is None else np.ascontiguousarray(biases, np.float32)
    sh = Shape4(shape[1], shape[0], shape[2], shape[3])
    st = Shape4(stride[0], stride[2], stride[1], stride[3])
    params = [act_dict[activation], int(use_bias), shape[1], shape[0], shape[2], shape[3], *stride]
    node = Node(lib.dR_Conv2d(input_node.graph.ptr, input_node.ptr, pointer(sh), pointer(st), act_dict[activation], int(use_bias)),
                input_node.graph, "Conv2D", params, [w, b])
    if w is not None:
        lib.dR_Conv2d_setVariables(node.ptr, _fptr(w), _fptr(b))
    if algo is not None:
        lib.dR_setConvAlgo(node.ptr, CONV_ALGO[algo])
    return node


def Fully_Connected(input_node, shape, activation, weights, biases=None):
    """shape = (Nin, Nout); weights [Nin, Nout] with rows in (H, W, C) flattening order."""
    use_bias = biases is not None
    w = None if weights is None else np.ascontiguousarray(weights, np.float32)
    b = None if biases is None else np.ascontiguousarray(biases, np.float32)
    sh = Shape2(shape[0], shape[1])
    node = Node(lib.dR_FullyConnected(input_node.graph.ptr, input_node.ptr, pointer(sh), act_dict[activation], int(use_bias)),
                input_node.graph, "FullyConnected", [act_dict[activation], int(use_bias), shape[0], shape[1]], [w, b])
    if w is not None:
        lib.dR_FullyConnected_setVariables(node.ptr, _fptr(w), _fptr(b))
    return node


def _ew1(input_node, op, scalar=0.0):
    return Node(lib.dR_ElemWise1Operation(input_node.graph.ptr, input_node.ptr, op, float(scalar)), input_node.graph, "ElemWise1Op", [op, scalar])


def _ew2(a, b, op):
    if a.graph is not b.graph:
        raise ValueError("DR Error: Inputs for element-wise operation are not in the same graph!")
    return Node(lib.dR_ElemWise2Operation(a.graph.ptr, a.ptr, b.ptr, op), a.graph, "ElemWise2Op", [op])


def Add_Scalar(input_node, scalar): return _ew1(input_node, 0, scalar)
def Sub_Scalar(input_node, scalar): return _ew1(input_node, 1, scalar)
def Mul_Scalar(input_node, scalar): return _ew1(input_node, 2, scalar)
def Div_Scalar(input_node, scalar): return _ew1(input_node, 3, scalar)
def Log(input_node): return _ew1(input_node, 4)
def Exp(input_node): return _ew1(input_node, 5)
def Sqrt(input_node): return _ew1(input_node, 6)
def Fill(input_node, scalar): return _ew1(input_node, 7, scalar)
def Pow_Scalar(input_node, scalar): return _ew1(input_node, 8, scalar)
def Add(a, b): return _ew2(a, b, 0)
def Sub(a, b): return _ew2(a, b, 1)
def Mul(a, b): return _ew2(a, b, 2)
def Div(a, b): return _ew2(a, b, 3)
def Pow(a, b): return _ew2(a, b, 4)


def Softmax(input_node):
    return Node(lib.dR_Softmax(input_node.graph.ptr, input_node.ptr), input_node.graph, "Softmax", [])


def Pooling(input_node, pooling_type, shape, stride):
    """shape / stride = (1, h, w, c) in the user's HWC sense (the reference passes them through
    untranslated, which is only right for square windows; here they are mapped to (., x, y, z))."""
    sh = Shape4(shape[0], shape[2], shape[1], shape[3])
    st = Shape4(stride[0], stride[2], stride[1], stride[3])
    return Node(lib.dR_Pooling(input_node.graph.ptr, input_node.ptr, pointer(sh), pointer(st), pool_dict[pooling_type]),
                input_node.graph, "Pooling", [pool_dict[pooling_type], *shape, *stride])


def Slice(input_node, origin, shape):
    o = _to_dr_shape3(input_node.graph.layout, list(origin))
    s = _to_dr_shape3(input_node.graph.layout, list(shape))
    return Node(lib.dR_Slice(input_node.graph.ptr, input_node.ptr, pointer(Shape4(*o, 0)), pointer(Shape4(*s, 0))),
                input_node.graph, "Slice", [*o, 0, *s, 0])


def Crop_Or_Pad(input_node, shape):
    s = _to_dr_shape3(input_node.graph.layout, list(shape))
    return Node(lib.dR_CropOrPad(input_node.graph.ptr, input_node.ptr, pointer(Shape3(*s))), input_node.graph, "CropOrPad", s)


def Concat(input_nodes, concat_dim):
    n = len(input_nodes)
    if n <= 1:
        raise ValueError("DR Error: Concat with one or less nodes not allowed!")
    graph = input_nodes[0].graph
    dr_dim = {"WHC": [0, 1, 2], "CHW": [2, 1, 0], "HWC": [1, 0, 2]}[graph.layout][concat_dim]
    ptrs = (c_void_p * n)()
    for i, nd in enumerate(input_nodes):
        if nd.graph is not graph:
            raise ValueError("DR Error: Inputs for Concat are not in the same graph!")
        ptrs[i] = nd.ptr
    return Node(lib.dR_Concat(graph.ptr, ptrs, n, dr_dim), graph, "Concat", [n, dr_dim])
