// Drives the C++ host mirror the way the reference's TransformerBlock drives LoraAdapter: read one projection case
// from a binary file, run Forward and Backward, write Y, dX, dA, dB back.  The GPU parity test compares the outputs
// with the CPU oracle.
//
// File layout (little endian): int32 qtype, N, K, T, rank; float alpha; int64 wbytes; then W bytes, X[T*K], dY[T*N],
// A[K*rank], B[rank*N].   Output: Y[T*N], dX[T*K], dA[K*rank], dB[rank*N] as fp32.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "glacier_tune_host.hpp"

using namespace Glacier::Tune;

template <class T>
static bool read_vec(FILE *f, std::vector<T> &v, size_t n) {
    v.resize(n);
    return fread(v.data(), sizeof(T), n, f) == n;
}

int main(int argc, char **argv) {
    if (argc < 3) {
        fprintf(stderr, "usage: %s case.bin out.bin\n", argv[0]);
        return 2;
    }
    FILE *f = fopen(argv[1], "rb");
    if (!f) return 2;
    int32_t hdr[5];
    float alpha;
    int64_t wbytes;
    if (fread(hdr, 4, 5, f) != 5 || fread(&alpha, 4, 1, f) != 1 || fread(&wbytes, 8, 1, f) != 1) return 2;
    const int qtype = hdr[0], N = hdr[1], K = hdr[2], T = hdr[3], rank = hdr[4];
    std::vector<uint8_t> W;
    std::vector<float> X, dY, A, B;
    if (!read_vec(f, W, (size_t)wbytes) || !read_vec(f, X, (size_t)T * K) || !read_vec(f, dY, (size_t)T * N) ||
        !read_vec(f, A, (size_t)K * rank) || !read_vec(f, B, (size_t)rank * N))
        return 2;
    fclose(f);
    try {
        GpuLoraEngine engine(0);
        const GgufType type = (GgufType)qtype;
        if (!engine.SupportsForwardGemm(type) || !engine.SupportsBackwardGemm(type)) return 3;
        gt_weight *dW = engine.UploadBaseWeight(type, W.data(), wbytes, N, K);
        LoraAdapter adapter(engine, K, N, rank, alpha);
        adapter.SetGpuBaseWeights(dW);
        adapter.SetParameters(A.data(), B.data());
        std::vector<float> Y((size_t)T * N), dX((size_t)T * K, 0.f), dA((size_t)K * rank), dB((size_t)rank * N);
        Tensor x(X.data(), T, K), y(Y.data(), T, N), dy(dY.data(), T, N), dx(dX.data(), T, K);
        adapter.Forward(type, x, y, T);
        adapter.Backward(type, dy, x, &dx);
        adapter.GetGradients(dA.data(), dB.data());
        FILE *o = fopen(argv[2], "wb");
        if (!o) return 2;
        fwrite(Y.data(), 4, Y.size(), o);
        fwrite(dX.data(), 4, dX.size(), o);
        fwrite(dA.data(), 4, dA.size(), o);
        fwrite(dB.data(), 4, dB.size(), o);
        fclose(o);
    } catch (const std::exception &ex) {
        fprintf(stderr, "host_example: %s\n", ex.what());
        return 1;
    }
    return 0;
}
