"""The TCP implementation of the network transport table (flagcx_net.h):
listen / connect / accept, one isend matched by one irecv, progressed by test()."""
import ctypes
import threading

from flagcx_b200.wrapper import default_library_path

HANDLE = 128
vp, sz = ctypes.c_void_p, ctypes.c_size_t
R = ctypes.c_int


class Props(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 64), ("pciPath", ctypes.c_char * 128), ("ptrSupport", ctypes.c_int), ("speedMbps", ctypes.c_int),
                ("port", ctypes.c_int), ("latencyUs", ctypes.c_float), ("maxComms", ctypes.c_int), ("maxRecvs", ctypes.c_int)]


class Adaptor(ctypes.Structure):
    F = ctypes.CFUNCTYPE
    _fields_ = [("name", ctypes.c_char_p), ("init", F(R)), ("devices", F(R, ctypes.POINTER(ctypes.c_int))),
                ("getProperties", F(R, ctypes.c_int, ctypes.POINTER(Props))), ("listen", F(R, ctypes.c_int, vp, ctypes.POINTER(vp))),
                ("connect", F(R, ctypes.c_int, vp, ctypes.POINTER(vp))), ("accept", F(R, vp, ctypes.POINTER(vp))),
                ("closeSend", F(R, vp)), ("closeRecv", F(R, vp)), ("closeListen", F(R, vp)),
                ("regMr", F(R, vp, vp, sz, ctypes.c_int, ctypes.POINTER(vp))),
                ("regMrDmaBuf", F(R, vp, vp, sz, ctypes.c_int, ctypes.c_uint64, ctypes.c_int, ctypes.POINTER(vp))),
                ("deregMr", F(R, vp, vp)), ("isend", F(R, vp, vp, sz, ctypes.c_int, vp, ctypes.POINTER(vp))),
                ("irecv", F(R, vp, ctypes.c_int, ctypes.POINTER(vp), ctypes.POINTER(sz), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(vp), ctypes.POINTER(vp))),
                ("iflush", F(R, vp, ctypes.c_int, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(vp), ctypes.POINTER(vp))),
                ("test", F(R, vp, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int))),
                ("write", vp), ("read", vp), ("signal", vp), ("getDevFromName", F(R, ctypes.c_char_p, ctypes.POINTER(ctypes.c_int)))]


def test_socket_adaptor_roundtrip(native_lib, monkeypatch):
    monkeypatch.setenv("FLAGCX_SOCKET_IFNAME", "lo")
    lib = ctypes.CDLL(native_lib)
    lib.flagcxGetNetAdaptor.restype = ctypes.POINTER(Adaptor)
    ad = lib.flagcxGetNetAdaptor().contents
    assert ad.name == b"socket" and ad.init() == 0
    n = ctypes.c_int()
    assert ad.devices(ctypes.byref(n)) == 0 and n.value == 1
    pr = Props()
    assert ad.getProperties(0, ctypes.byref(pr)) == 0 and pr.name == b"socket"
    handle = ctypes.create_string_buffer(HANDLE)
    lc, sc, rc = vp(), vp(), vp()
    assert ad.listen(0, handle, ctypes.byref(lc)) == 0
    t = threading.Thread(target=lambda: ad.accept(lc, ctypes.byref(rc)))
    t.start()
    assert ad.connect(0, handle, ctypes.byref(sc)) == 0
    t.join()
    payload = bytes(range(256)) * 4096  # 1 MiB: larger than the socket buffers, so test() has to be called repeatedly
    src = ctypes.create_string_buffer(payload, len(payload))
    dst = ctypes.create_string_buffer(len(payload))
    sreq, rreq = vp(), vp()
    assert ad.isend(sc, src, len(payload), 7, None, ctypes.byref(sreq)) == 0
    data = (vp * 1)(ctypes.cast(dst, vp))
    sizes = (sz * 1)(len(payload))
    tags = (ctypes.c_int * 1)(7)
    assert ad.irecv(rc, 1, data, sizes, tags, None, ctypes.byref(rreq)) == 0
    sdone = rdone = 0
    got = (ctypes.c_int * 1)()
    d = ctypes.c_int()
    for _ in range(1000000):
        if not sdone:
            assert ad.test(sreq, ctypes.byref(d), None) == 0
            sdone = d.value
        if not rdone:
            assert ad.test(rreq, ctypes.byref(d), got) == 0
            rdone = d.value
        if sdone and rdone:
            break
    assert sdone and rdone and got[0] == len(payload) and dst.raw == payload
    ad.closeSend(sc), ad.closeRecv(rc), ad.closeListen(lc)
