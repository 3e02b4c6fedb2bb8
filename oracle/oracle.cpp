// TEST INFRASTRUCTURE ONLY -- CPU restatement of Neureka's CPU-device implementation of the
// convolution / broadcast / elementwise path. It is the parity checker for the CUDA library and the
// timed CPU baseline; no product code may call into it.
//
// The reference is Java and cannot be executed where this file is built (no JVM), so every routine
// below restates the reference algorithm from its source and cites the file:line it follows.
// The restatement is pinned against the reference's own known-answer tests (tests/golden/).
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off -fno-fast-math -shared -fPIC -pthread
// (-ffp-contract=off because Java never fuses a*b+c; all accumulators have the tensor's own type.)
//
// View descriptor ("cfg"): int32[5*rank] laid out as NDConfiguration.asInlineArray()
//   [ shape | strides | indicesMap | offset | spread ]
// (src/main/java/neureka/ndim/config/NDConfiguration.java:335-345).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>
#include <algorithm>
#include <limits>

namespace {

constexpr int MAX_RANK = 16;

// ---------------------------------------------------------------------------------------------
// NDConfiguration + NDIterator
// ---------------------------------------------------------------------------------------------

// A view over the inline array. indexOfIndices follows
// src/main/java/neureka/ndim/config/types/sliced/SlicedNDConfiguration.java:103-109,
// indicesOfIndex follows :93-101.
struct NDC {
    int rank;
    const int32_t *shape, *strides, *imap, *offset, *spread;
    NDC(const int32_t* cfg, int r)
        : rank(r), shape(cfg), strides(cfg + r), imap(cfg + 2 * r), offset(cfg + 3 * r), spread(cfg + 4 * r) {}
    int64_t index_of_indices(const int* idx) const {
        int64_t index = 0;
        for (int i = 0; i < rank; i++)
            index += (int64_t(idx[i]) * spread[i] + offset[i]) * strides[i];
        return index;
    }
    void indices_of_index(int64_t index, int* idx) const {
        for (int i = 0; i < rank; i++) {
            idx[i] = int(index / imap[i]);
            index %= imap[i];
        }
    }
    int64_t size() const {
        int64_t s = 1;
        for (int i = 0; i < rank; i++) s *= shape[i];
        return s;
    }
    bool is_compact() const {  // NDConfiguration.java:386-392
        for (int i = 0; i < rank; i++)
            if (!(spread[i] == 1 || spread[i] == 0) || offset[i] != 0) return false;
        return true;
    }
};

// Layout.newStridesFor, NDConfiguration.java:106-129
void strides_for(const int32_t* shape, int rank, bool column_major, int* out) {
    int order[MAX_RANK];
    for (int i = 0; i < rank; i++) order[i] = rank - 1 - i;
    if (column_major && rank > 1) std::swap(order[0], order[1]);
    int prod = 1;
    for (int k = 0; k < rank; k++) {
        int i = order[k];
        out[i] = prod;
        prod *= shape[i];
    }
}

enum Layout { ROW_MAJOR, COLUMN_MAJOR, SYMMETRIC, UNSPECIFIC };

// NDConfiguration.getLayout, NDConfiguration.java:157-176
Layout layout_of(const NDC& c) {
    if (!c.is_compact()) return UNSPECIFIC;
    int rm[MAX_RANK], cm[MAX_RANK];
    strides_for(c.shape, c.rank, false, rm);
    strides_for(c.shape, c.rank, true, cm);
    bool has_rm_indices = std::equal(rm, rm + c.rank, c.imap);
    bool is_rm = std::equal(rm, rm + c.rank, c.strides) && has_rm_indices;
    bool is_cm = std::equal(cm, cm + c.rank, c.strides) && has_rm_indices;
    if (is_rm && is_cm) return SYMMETRIC;
    if (is_rm) return ROW_MAJOR;
    if (is_cm) return COLUMN_MAJOR;
    return UNSPECIFIC;
}

// NDConfiguration.isSimple, NDConfiguration.java:368-375
bool is_simple(const NDC& c) {
    Layout l = layout_of(c);
    int st[MAX_RANK];
    strides_for(c.shape, c.rank, l == COLUMN_MAJOR, st);
    return std::equal(st, st + c.rank, c.strides) && std::equal(st, st + c.rank, c.imap) && c.is_compact();
}

// NDIterator as implemented by SlicedNDIterator
// (src/main/java/neureka/ndim/iterator/types/sliced/SlicedNDIterator.java:25-46) with the
// increment of NDConfiguration.Utility.increment (NDConfiguration.java:436-450).
struct NDIter {
    NDC c;
    int idx[MAX_RANK];
    explicit NDIter(const NDC& conf) : c(conf) { std::memset(idx, 0, sizeof(idx)); }
    int shape(int a) const { return c.shape[a]; }
    int get(int a) const { return idx[a]; }
    void set(int a, int p) { idx[a] = p; }
    void set_all(const int* p) { std::memcpy(idx, p, sizeof(int) * c.rank); }
    int64_t i() const { return c.index_of_indices(idx); }
    int rank() const { return c.rank; }
    void increment() {
        int i = c.rank - 1;
        while (i >= 0 && i < c.rank) {
            if (idx[i] < c.shape[i]) {
                idx[i]++;
                if (idx[i] == c.shape[i]) { idx[i] = 0; i--; }
                else i = -1;
            } else i--;
        }
    }
};

// ---------------------------------------------------------------------------------------------
// CPU.JVMExecutor.threaded: contiguous split of [0, n) over the pool
// (src/main/java/neureka/devices/host/CPU.java:743-797). Only the partition matters for results.
// ---------------------------------------------------------------------------------------------
template <class F>
void threaded(int64_t n, int threads, F&& work) {
    if (threads <= 1 || n < 2) { work(int64_t(0), n); return; }
    int t = int(std::min<int64_t>(threads, n));
    std::vector<std::thread> pool;
    int64_t chunk = (n + t - 1) / t;
    for (int k = 0; k < t; k++) {
        int64_t s = k * chunk, e = std::min(n, s + chunk);
        if (s >= e) break;
        pool.emplace_back([=, &work] { work(s, e); });
    }
    for (auto& th : pool) th.join();
}

// ---------------------------------------------------------------------------------------------
// Convolution
// ---------------------------------------------------------------------------------------------

// AbstractCPUConvolution._convolve32/_convolve64
// (src/main/java/neureka/backend/main/implementations/convolution/AbstractCPUConvolution.java:245-316, :70-143)
// The operation is CPUConvolution's a*b (CPUConvolution.java:9-15).
template <class T>
void convolve(T* t0v, const NDC& c0, const T* t1v, const NDC& c1, const T* t2v, const NDC& c2,
              int64_t start, int64_t end) {
    NDIter t0(c0), t1(c1), t2(c2);
    int tmp[MAX_RANK];
    c0.indices_of_index(start, tmp);
    t0.set_all(tmp);
    const int rank = t0.rank();
    auto reset_axis = [&](int ri) {
        if (t1.shape(ri) == t2.shape(ri)) { t1.set(ri, t0.get(ri)); t2.set(ri, t0.get(ri)); }
        else if (t1.shape(ri) > t2.shape(ri)) { t1.set(ri, t0.get(ri)); t2.set(ri, 0); }
        else { t1.set(ri, 0); t2.set(ri, t0.get(ri)); }
    };
    for (int64_t i = start; i < end; i++) {
        int ri = 0;
        while (ri < rank) { reset_axis(ri); ri++; }
        T value = 0;
        bool running = true, incrementing = false;
        while (running) {
            ri = (ri == rank) ? 0 : ri;
            if (!incrementing) {
                value += t1v[t1.i()] * t2v[t2.i()];
                incrementing = true;
                ri = 0;
            } else {
                if (t1.get(ri) < t1.shape(ri) && t2.get(ri) < t2.shape(ri)) {
                    t1.set(ri, t1.get(ri) + 1);
                    t2.set(ri, t2.get(ri) + 1);
                    if (t1.get(ri) == t1.shape(ri) || t2.get(ri) == t2.shape(ri)) {
                        running = (ri != rank - 1);
                        reset_axis(ri);
                        ri++;
                    } else incrementing = false;
                } else ri++;
            }
        }
        t0v[t0.i()] = value;
        t0.increment();
    }
}

// AbstractCPUConvolution._deConvolve32/_deConvolve64 (AbstractCPUConvolution.java:319-408, :146-240)
template <class T>
void deconvolve(T* t0v, const NDC& c0, const T* t1v, const NDC& c1, const T* t2v, const NDC& c2,
                int64_t start, int64_t end) {
    NDIter t0(c0), t1(c1), t2(c2);
    int tmp[MAX_RANK];
    c0.indices_of_index(start, tmp);
    t0.set_all(tmp);
    const int rank = t0.rank();
    auto follow = [&](int ri) {
        t1.set(ri, t0.shape(ri) > t1.shape(ri) ? (t0.get(ri) - t2.get(ri)) : (t0.get(ri) + t2.get(ri)));
    };
    for (int64_t i = start; i < end; i++) {
        int ri = 0;
        while (ri < rank) {
            if (t2.get(ri) == t2.shape(ri)) { t1.set(ri, t0.get(ri)); t2.set(ri, 0); }
            else follow(ri);
            ri++;
        }
        T value = 0;
        bool running = true, incrementing = false;
        while (running) {
            ri = (ri == rank ? 0 : ri);
            if (!incrementing) {
                bool is_match = true;
                for (int rii = 0; rii < rank; rii++)
                    is_match = (t1.get(rii) < t1.shape(rii) && t1.get(rii) >= 0) && is_match;
                value += is_match ? t1v[t1.i()] * t2v[t2.i()] : T(0);
                incrementing = true;
                ri = 0;
            } else {
                if (t2.get(ri) < t2.shape(ri)) {
                    t2.set(ri, t2.get(ri) + 1);
                    if (t2.get(ri) == t2.shape(ri)) {
                        running = (ri != rank - 1);
                        t1.set(ri, t0.get(ri));
                        t2.set(ri, 0);
                        ri++;
                    } else {
                        follow(ri);
                        incrementing = false;
                    }
                } else ri++;
            }
        }
        t0v[t0.i()] = value;
        t0.increment();
    }
}

// SimpleCPUConvolution (implementations/convolution/SimpleCPUConvolution.java:11-235): the image
// fast path taken when d<0 and all three tensors are rank 2/3 and ROW_MAJOR or SYMMETRIC.
struct SimplePlan {
    bool ok = false;
    bool image_is_first = true;
    int width, height, kw, kh, rw, rh, batch;
};

bool simple_validate(const NDC& c) {  // SimpleCPUConvolution.java:225-233
    if (c.rank != 2 && c.rank != 3) return false;
    Layout l = layout_of(c);
    return l == ROW_MAJOR || l == SYMMETRIC;
}

bool simple_try(const NDC& image, const NDC& kernel, const NDC& result, SimplePlan& p) {  // :35-64
    if (!simple_validate(image) || !simple_validate(kernel) || !simple_validate(result)) return false;
    int batch = image.rank == 3 ? image.shape[0] : 1;
    int so = image.rank == 3 ? 1 : 0;
    // Mixed ranks index out of bounds in the reference (exception swallowed => not suitable).
    if (kernel.rank < so + 2) return false;
    p.width = image.shape[so + 1];
    p.height = image.shape[so + 0];
    p.kw = kernel.shape[so + 1];
    p.kh = kernel.shape[so + 0];
    int kbatch = kernel.rank == 3 ? kernel.shape[0] : 1;
    p.rw = p.width - p.kw + 1;
    p.rh = p.height - p.kh + 1;
    p.batch = batch;
    if (kbatch > 1) return false;
    if (int64_t(batch) * p.rh * p.rw != result.size()) return false;
    return true;
}

// Constructor order of SimpleCPUConvolution.java:15-26: (in1 image) first, then (in2 image); the
// last attempt that succeeds wins.
SimplePlan simple_plan(const NDC& in1, const NDC& in2, const NDC& out) {
    SimplePlan best, p;
    if (simple_try(in1, in2, out, p)) { best = p; best.ok = true; best.image_is_first = true; }
    if (simple_try(in2, in1, out, p)) { best = p; best.ok = true; best.image_is_first = false; }
    return best;
}

template <class T>
void simple_conv_batch(const SimplePlan& p, const T* image, const T* kernel, T* result, int bi) {  // :143-159
    int64_t image_off = int64_t(bi) * p.width * p.height;
    int64_t result_off = int64_t(bi) * p.rw * p.rh;
    for (int y = 0; y < p.rh; y++)
        for (int x = 0; x < p.rw; x++) {
            T sum = 0;
            for (int ky = 0; ky < p.kh; ky++)
                for (int kx = 0; kx < p.kw; kx++)
                    sum += image[image_off + int64_t(y + ky) * p.width + (x + kx)] * kernel[ky * p.kw + kx];
            result[result_off + int64_t(y) * p.rw + x] = sum;
        }
}

// AbstractCPUConvolution.run (AbstractCPUConvolution.java:16-36)
template <class T>
int conv_run(T* drn, const int32_t* cfg0, const T* s1, const int32_t* cfg1, const T* s2, const int32_t* cfg2,
             int rank, int d, int threads, int allow_simple) {
    NDC c0(cfg0, rank), c1(cfg1, rank), c2(cfg2, rank);
    if (allow_simple && d < 0) {
        SimplePlan p = simple_plan(c1, c2, c0);
        if (p.ok) {
            const T* image = p.image_is_first ? s1 : s2;
            const T* kernel = p.image_is_first ? s2 : s1;
            int work = p.rh * p.rw;
            if (work < 1000 || threads <= 1)  // SimpleCPUConvolution.java:135-141
                for (int bi = 0; bi < p.batch; bi++) simple_conv_batch(p, image, kernel, drn, bi);
            else
                threaded(p.batch, threads, [&](int64_t s, int64_t e) {
                    for (int64_t bi = s; bi < e; bi++) simple_conv_batch(p, image, kernel, drn, int(bi));
                });
            return 1;
        }
    }
    threaded(c0.size(), threads, [&](int64_t s, int64_t e) {
        if (d < 0) convolve<T>(drn, c0, s1, c1, s2, c2, s, e);
        else deconvolve<T>(drn, c0, s1, c1, s2, c2, s, e);
    });
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Binary scalar kernels (value / derivative 0 / derivative 1), per implementation family
// ---------------------------------------------------------------------------------------------
enum Op { OP_ADD = 0, OP_SUB = 1, OP_MUL = 2, OP_DIV = 3, OP_MOD = 4, OP_POW = 5, OP_IDY = 6, OP_TEST_MUL = 7 };

inline float jmod(float a, float b) { return std::fmod(a, b); }
inline double jmod(double a, double b) { return std::fmod(a, b); }

// CPUBroadcast{Addition,Subtraction,Multiplication,Division,Modulo,Power}.java (each :10-32).
// d selects _getFun (d<0), _getDeriveAt0 (d==0), _getDeriveAt1 (d==1), CPUBroadcast.java:41-42.
template <class T>
T broadcast_fun(int op, int d, T a, T b) {
    switch (op) {
        case OP_ADD: return a + b;  // derivatives are _getFun as well (CPUBroadcastAddition.java:19-21)
        case OP_SUB: return d == 0 ? a + b : a - b;  // CPUBroadcastSubtraction.java:13-31
        case OP_MUL: return d == 0 ? b : (d == 1 ? a : a * b);
        case OP_DIV:
            if (d == 0) return T(1) / b;
            if (d == 1) return T(-(double(a) / std::pow(double(b), 2)));
            return a / b;
        case OP_MOD:
            if (d == 0) return T(1) / b;
            if (d == 1) return T(-(double(a) / std::pow(double(b), 2)));
            return jmod(a, b);
        case OP_POW:
            if (d == 0) return T(double(a) * std::pow(double(a), double(b) - 1));  // sic, CPUBroadcastPower.java:22-23
            if (d == 1) return T(std::pow(double(a), double(b)) * std::log(double(a)));
            return T(std::pow(double(a), double(b)));
        case OP_TEST_MUL: return a * b;  // TestBroadcast of src/test/java/testutility/UnitTester_Tensor.java:414-433
    }
    return std::numeric_limits<T>::quiet_NaN();
}
// Note for OP_POW d==0 with T=float: the Java float overload computes b-1 in float first
// ("Math.pow( a, b - 1 )" with float a,b). Handled by the specialisation below.
template <>
float broadcast_fun<float>(int op, int d, float a, float b) {
    switch (op) {
        case OP_ADD: return a + b;
        case OP_SUB: return d == 0 ? a + b : a - b;
        case OP_MUL: return d == 0 ? b : (d == 1 ? a : a * b);
        case OP_DIV:
            if (d == 0) return 1 / b;
            if (d == 1) return float(-(double(a) / std::pow(double(b), 2)));
            return a / b;
        case OP_MOD:
            if (d == 0) return 1 / b;
            if (d == 1) return float(-(double(a) / std::pow(double(b), 2)));
            return jmod(a, b);
        case OP_POW:
            if (d == 0) return float(double(a) * std::pow(double(a), double(b - 1)));
            if (d == 1) return float(std::pow(double(a), double(b)) * std::log(double(a)));
            return float(std::pow(double(a), double(b)));
        case OP_TEST_MUL: return a * b;
    }
    return std::numeric_limits<float>::quiet_NaN();
}

// CPUBiElementWise{Addition,...,Power}.java (each :9-35)
inline double bielem_fun(int op, int d, double a, double b) {
    switch (op) {
        case OP_ADD: return d >= 0 ? 1.0 : a + b;
        case OP_SUB: return d == 0 ? 1.0 : (d == 1 ? -1.0 : a - b);
        case OP_MUL: return d == 0 ? b : (d == 1 ? a : a * b);
        case OP_DIV:
            if (d == 0) return 1.0 / b;
            if (d == 1) return -a / std::pow(b, 2);
            return a / b;
        case OP_MOD:
            if (d == 0) return 1.0 / b;
            if (d == 1) return -a / std::pow(b, 2);
            return jmod(a, b);
        case OP_POW:
            if (d == 0) return b * std::pow(a, b - 1);
            if (d == 1) return std::pow(a, b) * std::log(a);
            return std::pow(a, b);
    }
    return std::numeric_limits<double>::quiet_NaN();
}
inline float bielem_fun(int op, int d, float a, float b) {
    switch (op) {
        case OP_ADD: return d >= 0 ? 1.0f : a + b;
        case OP_SUB: return d == 0 ? 1.0f : (d == 1 ? -1.0f : a - b);
        case OP_MUL: return d == 0 ? b : (d == 1 ? a : a * b);
        case OP_DIV:
            if (d == 0) return 1.0f / b;
            if (d == 1) return float(-(double(a) / std::pow(double(b), 2)));
            return a / b;
        case OP_MOD:
            if (d == 0) return 1.0f / b;
            if (d == 1) return float(-(double(a) / std::pow(double(b), 2)));
            return jmod(a, b);
        case OP_POW:
            if (d == 0) return float(double(b) * std::pow(double(a), double(b - 1)));
            if (d == 1) return float(std::pow(double(a), double(b)) * std::log(double(a)));
            return float(std::pow(double(a), double(b)));
    }
    return std::numeric_limits<float>::quiet_NaN();
}

// CPUScalarBroadcast{Addition,Subtraction,Multiplication,Division,Modulo,Identity}.java and
// CPUScalaBroadcastPower.java: tensor (a) op scalar (b).
inline double scalar_fun(int op, int d, double a, double b) {
    switch (op) {
        case OP_ADD: return d >= 0 ? 1.0 : a + b;
        case OP_SUB: return d == 0 ? 1.0 : (d == 1 ? -1.0 : a - b);
        case OP_MUL: return d == 0 ? b : (d == 1 ? a : a * b);
        case OP_DIV:
            if (d == 0) return 1 / b;
            if (d == 1) return -(a / std::pow(b, 2));
            return a / b;
        case OP_MOD:
            if (d == 0) return 1 / b;
            if (d == 1) return -(a / std::pow(b, 2));
            return jmod(a, b);
        case OP_POW:
            if (d == 0) return b * std::pow(a, b - 1);
            if (d == 1) return std::pow(a, b) * std::log(a);
            return std::pow(a, b);
        case OP_IDY: return b;
    }
    return std::numeric_limits<double>::quiet_NaN();
}
inline float scalar_fun(int op, int d, float a, float b) {
    switch (op) {
        case OP_ADD: return d >= 0 ? 1.0f : a + b;
        case OP_SUB: return d == 0 ? 1.0f : (d == 1 ? -1.0f : a - b);
        case OP_MUL: return d == 0 ? b : (d == 1 ? a : a * b);
        case OP_DIV:
            if (d == 0) return 1 / b;
            if (d == 1) return float(-(double(a) / std::pow(double(b), 2)));
            return a / b;
        case OP_MOD:
            if (d == 0) return 1 / b;
            if (d == 1) return float(-(double(a) / std::pow(double(b), 2)));
            return jmod(a, b);
        case OP_POW:
            if (d == 0) return float(double(b) * std::pow(double(a), double(b - 1)));
            if (d == 1) return float(std::pow(double(a), double(b)) * std::log(double(a)));
            return float(std::pow(double(a), double(b)));
        case OP_IDY: return b;
    }
    return std::numeric_limits<float>::quiet_NaN();
}

// ---------------------------------------------------------------------------------------------
// Broadcast: CPUBroadcast._broadcastF32/_broadcastF64
// (src/main/java/neureka/backend/main/implementations/broadcast/CPUBroadcast.java:62-160, :164-260)
// ---------------------------------------------------------------------------------------------
template <class T>
void broadcast(T* t0v, const NDC& c0, const T* t1v, const NDC& c1, const T* t2v, const NDC& c2,
               int op, int d, int64_t i, int64_t end) {
    const int32_t *t0Shp = c0.shape, *t1Shp = c1.shape, *t2Shp = c2.shape;
    const int rank = c0.rank;
    NDIter t0(c0), t1(c1), t2(c2);
    int tmp[MAX_RANK];
    c0.indices_of_index(i, tmp);
    t0.set_all(tmp);
    t1.set_all(tmp);
    if (d < 0) {
        while (i < end) {
            int ri = 0;
            while (ri < rank) {
                if (t1Shp[ri] == t2Shp[ri]) { t1.set(ri, t0.get(ri)); t2.set(ri, t0.get(ri)); }
                else if (t1Shp[ri] > t2Shp[ri]) { t1.set(ri, t0.get(ri)); t2.set(ri, 0); }
                else if (t1Shp[ri] < t2Shp[ri]) { t1.set(ri, 0); t2.set(ri, t0.get(ri)); }
                ri++;
            }
            t0v[t0.i()] = broadcast_fun<T>(op, d, t1v[t1.i()], t2v[t2.i()]);
            t0.increment();
            i++;
        }
    } else {
        while (i < end) {
            int ri = 0;
            while (ri < rank) {
                if (t0Shp[ri] == t1Shp[ri]) {
                    t1.set(ri, t0.get(ri));
                    t2.set(ri, t0.get(ri));
                    if (t2Shp[ri] == 1) t2.set(ri, 0);
                    else t2.set(ri, t0.get(ri));
                } else if (t0Shp[ri] > t1Shp[ri]) {
                    t1.set(ri, 0);
                    t2.set(ri, t0.get(ri));
                }
                ri++;
            }
            T value = 0;
            bool running = true, incrementing = false;
            while (running) {
                ri = (ri == rank ? 0 : ri);
                if (!incrementing) {
                    value += broadcast_fun<T>(op, d, t1v[t1.i()], t2v[t2.i()]);
                    incrementing = true;
                    ri = 0;
                } else {
                    if (t0Shp[ri] < t1Shp[ri]) {
                        t1.set(ri, t1.get(ri) + 1);
                        t2.set(ri, t2.get(ri) + 1);
                        if (t1.get(ri) == t1Shp[ri]) {
                            t1.set(ri, 0);
                            t2.set(ri, 0);
                            running = (ri != rank - 1);
                            ri++;
                        } else incrementing = false;
                    } else {
                        running = (ri != rank - 1);
                        ri++;
                    }
                }
            }
            t0v[t0.i()] = value;
            t0.increment();
            i++;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// BiElementwise: CPUBiElementWise._newWorkloadF32/_newWorkloadF64
// (src/main/java/neureka/backend/main/implementations/elementwise/CPUBiElementWise.java:56-140)
// ---------------------------------------------------------------------------------------------
template <class T>
void bielementwise(T* t0v, const NDC& c0, const T* t1v, const NDC& c1, const T* t2v, const NDC& c2,
                   int op, int d, int64_t i, int64_t end) {
    if (is_simple(c0) && is_simple(c1) && is_simple(c2)) {
        for (; i < end; i++) t0v[i] = bielem_fun(op, d, t1v[i], t2v[i]);
        return;
    }
    NDIter t0(c0), t1(c1), t2(c2);
    int tmp[MAX_RANK];
    c0.indices_of_index(i, tmp); t0.set_all(tmp);
    c1.indices_of_index(i, tmp); t1.set_all(tmp);
    c2.indices_of_index(i, tmp); t2.set_all(tmp);
    while (i < end) {
        t0v[t0.i()] = bielem_fun(op, d, t1v[t1.i()], t2v[t2.i()]);
        t0.increment(); t1.increment(); t2.increment();
        i++;
    }
}

// ---------------------------------------------------------------------------------------------
// Scalar broadcast: CPUScalarBroadcast._workloadFor
// (src/main/java/neureka/backend/main/implementations/broadcast/CPUScalarBroadcast.java:29-75)
// ---------------------------------------------------------------------------------------------
template <class T>
void scalar_broadcast(T* t0v, const NDC& c0, const T* t1v, const NDC& c1, T value,
                      int op, int d, int64_t i, int64_t end) {
    NDIter t0(c0), src(c1);
    int tmp[MAX_RANK];
    c0.indices_of_index(i, tmp); t0.set_all(tmp);
    c1.indices_of_index(i, tmp); src.set_all(tmp);
    while (i < end) {
        t0v[t0.i()] = scalar_fun(op, d, t1v[src.i()], value);
        t0.increment(); src.increment();
        i++;
    }
}

// ---------------------------------------------------------------------------------------------
// The 23 scalar functions (src/main/java/neureka/backend/main/implementations/fun/*.java).
// Order = ids below. F32 follows each class's float overload; where a class has none, the default
// of CPUFun.invoke(float) applies: evaluate the double formula and cast
// (implementations/fun/api/CPUFun.java:7-9).
// ---------------------------------------------------------------------------------------------
enum Fun {
    F_ABS = 0, F_CBRT, F_COS, F_EXP, F_GASU, F_GATU, F_GAUS, F_FAST_GAUS, F_GELU, F_IDY, F_LOG10, F_LN,
    F_QUAD, F_RELU, F_SELU, F_SILU, F_SIG, F_SIN, F_SOFTPLUS, F_SOFTSIGN, F_SQRT, F_TANH, F_FAST_TANH,
    F_COUNT
};

// FunUtil.invSqrt (implementations/fun/FunUtil.java:8-29)
inline double inv_sqrt(double x) {
    double xhalf = 0.5 * x;
    int64_t i;
    std::memcpy(&i, &x, 8);
    i = 0x5fe6ec85e7de30daLL - (i >> 1);
    std::memcpy(&x, &i, 8);
    x *= (1.5 - xhalf * x * x);
    x *= (1.5 - xhalf * x * x);
    x *= (1.5 - xhalf * x * x);
    x *= (1.5 - xhalf * x * x);
    return x;
}
inline float inv_sqrt(float x) {
    float xhalf = 0.5f * x;
    int32_t i;
    std::memcpy(&i, &x, 4);
    i = 0x5f3759df - (i >> 1);
    std::memcpy(&x, &i, 4);
    x *= (1.5f - xhalf * x * x);
    x *= (1.5f - xhalf * x * x);
    return x;
}

constexpr double SELU_ALPHA = 1.6732632423543772848170429916717;  // ScalarSeLU.java:9-10
constexpr double SELU_SCALE = 1.0507009873554804934193349852946;

inline double sig64(double x) { return 1.0 / (1.0 + std::exp(-x)); }                // ScalarSigmoid.java:39
inline double tanh64(double x) { return 2 / (1 + std::exp(-x * 2)) - 1; }           // ScalarTanh.java:39
inline float tanh32(float x) { return float(2 / (1 + std::exp(double(-x * 2))) - 1); }  // ScalarTanh.java:40
inline double softsign64(double x) { return x / (1.0 + std::fabs(x)); }             // ScalarSoftsign.java:46
inline float softsign32(float x) { return x / (1.0f + std::fabs(x)); }              // ScalarSoftsign.java:47
inline double selu64(double x) {                                                    // ScalarSeLU.java:66-70
    if (x > 0) return SELU_SCALE * x;
    else if (x <= 0) return SELU_SCALE * SELU_ALPHA * (std::exp(x) - 1);
    else return std::numeric_limits<float>::quiet_NaN();
}

double fun64(int f, bool derive, double x) {
    if (!derive) switch (f) {
        case F_ABS: return std::fabs(x);
        case F_CBRT: return std::cbrt(x);
        case F_COS: return std::cos(x);
        case F_EXP: return std::exp(x);
        case F_GASU: return softsign64(x * x * x);
        case F_GATU: return tanh64(x * x * x);
        case F_GAUS: return std::exp(-(x * x));
        case F_FAST_GAUS: return 1 / (1 + x * x);
        case F_GELU: return x * sig64(x * 1.702);
        case F_IDY: return x;
        case F_LOG10: return std::log10(x);
        case F_LN: return std::log(x);
        case F_QUAD: return x * x;
        case F_RELU: return x >= 0 ? x : x * .01;
        case F_SELU: return selu64(x);
        case F_SILU: return x * sig64(x);
        case F_SIG: return sig64(x);
        case F_SIN: return std::sin(x);
        case F_SOFTPLUS: return std::log(1.0 + std::exp(x));
        case F_SOFTSIGN: return softsign64(x);
        case F_SQRT: return std::sqrt(x);
        case F_TANH: return tanh64(x);
        case F_FAST_TANH: return x * inv_sqrt(1.0 + x * x);
    }
    else switch (f) {
        case F_ABS: return x < 0 ? -1.0 : 1.0;
        case F_CBRT: return 1 / (3 * std::pow(x, 2.0 / 3.0));
        case F_COS: return -std::sin(x);
        case F_EXP: return std::exp(x);
        case F_GASU: { double x2 = x * x, x6 = x2 * x2 * x2; return 3.0 * x2 / (2.0 * x2 * std::fabs(x) + x6 + 1.0); }
        case F_GATU: {
            double x2 = x * x, x3 = x2 * x, temp = 3 * x2, tanh2 = std::pow(tanh64(x3), 2);
            return -temp * tanh2 + temp;
        }
        case F_GAUS: return -2 * x * std::exp(-(x * x));
        case F_FAST_GAUS: { double x2 = x * x; return -2 * x / (x2 * x2 + 2 * x2 + 1); }
        case F_GELU: { double s = sig64(x * 1.702), ds = s * (1.0 - s); return s + ds * x * 1.702; }
        case F_IDY: return 1;
        case F_LOG10: return 1 / (x * std::log(10.0));
        case F_LN: return 1.0 / x;
        case F_QUAD: return 2 * x;
        case F_RELU: return x >= 0 ? 1 : .01;
        case F_SELU:
            if (x > 0) return SELU_SCALE;
            else if (x <= 0) return SELU_SCALE * SELU_ALPHA * std::exp(x);
            else return std::numeric_limits<double>::quiet_NaN();
        case F_SILU: { double s = sig64(x); return s + (x * s * (1.0 - s)); }
        case F_SIG: { double s = sig64(x); return s * (1 - s); }
        case F_SIN: return std::cos(x);
        case F_SOFTPLUS: return 1.0 / (1.0 + std::exp(-x));
        case F_SOFTSIGN: return 1.0 / (2.0 * std::fabs(x) + x * x + 1.0);
        case F_SQRT: return 0.5 * inv_sqrt(x);
        case F_TANH: return 1 - std::pow(tanh64(x), 2);
        case F_FAST_TANH: { double t1 = x * x, t2 = std::sqrt(1 + t1); return 1 / (t1 * t2 + t2); }
    }
    return std::numeric_limits<double>::quiet_NaN();
}

float fun32(int f, bool derive, float x) {
    if (!derive) switch (f) {
        case F_ABS: return std::fabs(x);
        case F_CBRT: return float(std::cbrt(double(x)));
        case F_EXP: return float(std::exp(double(x)));
        case F_GASU: return softsign32(x * x * x);
        case F_GATU: return tanh32(x * x * x);
        case F_FAST_GAUS: return 1 / (1 + x * x);
        case F_GELU: return float(double(x) * sig64(double(x) * 1.702));
        case F_IDY: return x;
        case F_LOG10: return float(std::log10(double(x)));
        case F_QUAD: return x * x;
        case F_RELU: return x >= 0 ? x : x * .01f;
        case F_SELU: return float(selu64(double(x)));
        case F_SILU: return float(double(x) * sig64(double(x)));
        case F_SIG: return float(sig64(double(x)));
        case F_SOFTSIGN: return softsign32(x);
        case F_SQRT: return float(std::sqrt(double(x)));
        case F_TANH: return tanh32(x);
        case F_FAST_TANH: return x * inv_sqrt(1.0f + x * x);
        default: return float(fun64(f, false, double(x)));  // cos, gaus, ln, sin, softplus
    }
    else switch (f) {
        case F_ABS: return x < 0.0f ? -1.0f : 1.0f;
        case F_CBRT: return 1 / (3 * float(std::pow(double(x), double(2.0f / 3.0f))));
        case F_EXP: return float(std::exp(double(x)));
        case F_GASU: { float x2 = x * x, x6 = x2 * x2 * x2; return 3.0f * x2 / (2.0f * x2 * std::fabs(x) + x6 + 1.0f); }
        case F_GATU: {
            float x2 = x * x, x3 = x2 * x, temp = 3 * x2;
            float tanh2 = float(std::pow(double(tanh32(x3)), 2));
            return -temp * tanh2 + temp;
        }
        case F_FAST_GAUS: { float x2 = x * x; return -2 * x / (x2 * x2 + 2 * x2 + 1); }
        case F_GELU: { float s = float(sig64(double(x) * 1.702)); float ds = s * (1.0f - s); return s + ds * x * 1.702f; }
        case F_IDY: return 1;
        case F_LOG10: return 1 / (x * float(std::log(10.0)));
        case F_LN: return 1.0f / x;
        case F_QUAD: return 2 * x;
        case F_RELU: return x >= 0 ? 1.0f : .01f;
        case F_SELU:
            if (x > 0) return float(SELU_SCALE);
            else if (x <= 0) return float(SELU_SCALE * SELU_ALPHA * std::exp(double(x)));
            else return std::numeric_limits<float>::quiet_NaN();
        case F_SILU: { float s = float(sig64(double(x))); return s + (x * s * (1.0f - s)); }
        case F_SIG: { float s = float(sig64(double(x))); return s * (1 - s); }
        case F_SOFTSIGN: return 1.0f / (2.0f * std::fabs(x) + x * x + 1.0f);
        case F_SQRT: return 0.5f * inv_sqrt(x);
        case F_TANH: return float(1 - std::pow(double(tanh32(x)), 2));
        case F_FAST_TANH: { float t1 = x * x; float t2 = float(std::sqrt(double(1 + t1))); return 1 / (t1 * t2 + t2); }
        default: return float(fun64(f, true, double(x)));  // cos, gaus, sin, softplus
    }
}

inline double fun_any(int f, bool derive, double x) { return fun64(f, derive, x); }
inline float fun_any(int f, bool derive, float x) { return fun32(f, derive, x); }

// CPUElementwiseFunction._workloadFor
// (src/main/java/neureka/backend/main/implementations/elementwise/CPUElementwiseFunction.java:30-116)
template <class T>
void unary(T* t0v, const NDC& c0, const T* t1v, const NDC& c1, int f, int d, int64_t i, int64_t end) {
    bool derive = d >= 0;
    if (is_simple(c0) && is_simple(c1)) {
        for (; i < end; i++) t0v[i] = fun_any(f, derive, t1v[i]);
        return;
    }
    NDIter t0(c0), t1(c1);
    int tmp[MAX_RANK];
    c0.indices_of_index(i, tmp);
    t0.set_all(tmp);
    t1.set_all(tmp);  // both positioned from the drain's indices (:105-106)
    while (i < end) {
        t0v[t0.i()] = fun_any(f, derive, t1v[t1.i()]);
        t0.increment(); t1.increment();
        i++;
    }
}

// CPUSum._runRecursively (src/main/java/neureka/backend/main/operations/other/internal/CPUSum.java:26-76)
template <class T>
T sum_recursive(const T* in, int64_t size) {
    const int RTS = 128;
    if (size == 1) return in[0];
    int64_t n = (size + RTS - 1) / RTS;
    std::vector<T> out(n);
    for (int64_t ni = 0; ni < n; ni++) {
        int64_t off = ni * RTS, limit = std::min(off + RTS, size);
        T value = 0;
        for (int64_t k = off; k < limit; k++) value += in[k];
        out[ni] = value;
    }
    if (n > 1) return sum_recursive(out.data(), n);
    return out[0];
}

// ---------------------------------------------------------------------------------------------
// java.util.Random-compatible generator
// (constants: implementations/elementwise/CPURandomization.java:12-15; stepping :286-307;
//  polar Gaussian :265-284)
// ---------------------------------------------------------------------------------------------
constexpr uint64_t J_MULT = 0x5DEECE66DULL, J_ADD = 0xBULL, J_MASK = (1ULL << 48) - 1;
inline uint64_t j_next_seed(uint64_t s) { return (s * J_MULT + J_ADD) & J_MASK; }
inline int32_t j_next(int bits, uint64_t seed) { return int32_t(int64_t(seed) >> (48 - bits)); }
inline double j_next_double(uint64_t s1, uint64_t s2) {
    return double((int64_t(j_next(26, s1)) << 27) + j_next(27, s2)) * 0x1.0p-53;
}
// CPURandomization.gaussianFrom (:265-284); 'seed' is used as given (no initial scramble).
void gaussian_from(uint64_t seed, double* out) {
    double v1, v2, s;
    seed &= J_MASK;  // the first _nextSeed masks anyway; kept explicit for clarity
    do {
        uint64_t s1 = j_next_seed(seed), s2 = j_next_seed(s1), s3 = j_next_seed(s2), s4 = j_next_seed(s3);
        v1 = 2 * j_next_double(s1, s2) - 1;
        v2 = 2 * j_next_double(s3, s4) - 1;
        s = v1 * v1 + v2 * v2;
        seed = s4;
    } while (s >= 1 || s == 0);
    double multiplier = std::sqrt(-2 * std::log(s) / s);
    out[0] = v1 * multiplier;
    out[1] = v2 * multiplier;
}

template <class T>
int run3(int kind, int dtype_rank, T* drn, const int32_t* cfg0, const T* a, const int32_t* cfg1,
         const T* b, const int32_t* cfg2, int op, int d, int threads) {
    int rank = dtype_rank;
    NDC c0(cfg0, rank), c1(cfg1, rank), c2(cfg2, rank);
    threaded(c0.size(), threads, [&](int64_t s, int64_t e) {
        if (kind == 0) broadcast<T>(drn, c0, a, c1, b, c2, op, d, s, e);
        else bielementwise<T>(drn, c0, a, c1, b, c2, op, d, s, e);
    });
    return 0;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// C entry points (ctypes). dtype: 0 = F32, 1 = F64.
// ---------------------------------------------------------------------------------------------
extern "C" {

int orc_conv(int dtype, int rank, void* drn, const int32_t* cfg0, const void* s1, const int32_t* cfg1,
             const void* s2, const int32_t* cfg2, int d, int threads, int allow_simple) {
    if (rank > MAX_RANK) return -1;
    if (dtype == 0) return conv_run<float>((float*)drn, cfg0, (const float*)s1, cfg1, (const float*)s2, cfg2, rank, d, threads, allow_simple);
    if (dtype == 1) return conv_run<double>((double*)drn, cfg0, (const double*)s1, cfg1, (const double*)s2, cfg2, rank, d, threads, allow_simple);
    return -1;
}

// Evaluates only drain elements [start, end) with the general nd algorithm (d<0: _convolve, else
// _deConvolve) -- used to spot-check very large configurations.
int orc_conv_range(int dtype, int rank, void* drn, const int32_t* cfg0, const void* s1, const int32_t* cfg1,
                   const void* s2, const int32_t* cfg2, int d, int64_t start, int64_t end) {
    if (rank > MAX_RANK) return -1;
    NDC c0(cfg0, rank), c1(cfg1, rank), c2(cfg2, rank);
    if (dtype == 0) {
        if (d < 0) convolve<float>((float*)drn, c0, (const float*)s1, c1, (const float*)s2, c2, start, end);
        else deconvolve<float>((float*)drn, c0, (const float*)s1, c1, (const float*)s2, c2, start, end);
    } else if (dtype == 1) {
        if (d < 0) convolve<double>((double*)drn, c0, (const double*)s1, c1, (const double*)s2, c2, start, end);
        else deconvolve<double>((double*)drn, c0, (const double*)s1, c1, (const double*)s2, c2, start, end);
    } else return -1;
    return 0;
}

int orc_simple_conv_suitable(int rank, const int32_t* cfg0, const int32_t* cfg1, const int32_t* cfg2) {
    NDC c0(cfg0, rank), c1(cfg1, rank), c2(cfg2, rank);
    return simple_plan(c1, c2, c0).ok ? 1 : 0;
}

int orc_broadcast(int dtype, int rank, void* drn, const int32_t* cfg0, const void* a, const int32_t* cfg1,
                  const void* b, const int32_t* cfg2, int op, int d, int threads) {
    if (rank > MAX_RANK) return -1;
    if (dtype == 0) return run3<float>(0, rank, (float*)drn, cfg0, (const float*)a, cfg1, (const float*)b, cfg2, op, d, threads);
    if (dtype == 1) return run3<double>(0, rank, (double*)drn, cfg0, (const double*)a, cfg1, (const double*)b, cfg2, op, d, threads);
    return -1;
}

int orc_bielementwise(int dtype, int rank, void* drn, const int32_t* cfg0, const void* a, const int32_t* cfg1,
                      const void* b, const int32_t* cfg2, int op, int d, int threads) {
    if (rank > MAX_RANK) return -1;
    if (dtype == 0) return run3<float>(1, rank, (float*)drn, cfg0, (const float*)a, cfg1, (const float*)b, cfg2, op, d, threads);
    if (dtype == 1) return run3<double>(1, rank, (double*)drn, cfg0, (const double*)a, cfg1, (const double*)b, cfg2, op, d, threads);
    return -1;
}

int orc_scalar_broadcast(int dtype, int rank, void* drn, const int32_t* cfg0, const void* a, const int32_t* cfg1,
                         double value, int op, int d, int threads) {
    if (rank > MAX_RANK) return -1;
    NDC c0(cfg0, rank), c1(cfg1, rank);
    threaded(c0.size(), threads, [&](int64_t s, int64_t e) {
        if (dtype == 0) scalar_broadcast<float>((float*)drn, c0, (const float*)a, c1, float(value), op, d, s, e);
        else scalar_broadcast<double>((double*)drn, c0, (const double*)a, c1, value, op, d, s, e);
    });
    return 0;
}

int orc_unary(int dtype, int rank, void* drn, const int32_t* cfg0, const void* a, const int32_t* cfg1,
              int fun, int d, int threads) {
    if (rank > MAX_RANK || fun < 0 || fun >= F_COUNT) return -1;
    NDC c0(cfg0, rank), c1(cfg1, rank);
    threaded(c0.size(), threads, [&](int64_t s, int64_t e) {
        if (dtype == 0) unary<float>((float*)drn, c0, (const float*)a, c1, fun, d, s, e);
        else unary<double>((double*)drn, c0, (const double*)a, c1, fun, d, s, e);
    });
    return 0;
}

double orc_fun64(int fun, int derive, double x) { return fun64(fun, derive != 0, x); }
float orc_fun32(int fun, int derive, float x) { return fun32(fun, derive != 0, x); }

double orc_sum(int dtype, const void* in, int64_t n) {
    if (dtype == 0) return double(sum_recursive<float>((const float*)in, n));
    return sum_recursive<double>((const double*)in, n);
}

int orc_layout(int rank, const int32_t* cfg) { return int(layout_of(NDC(cfg, rank))); }
int orc_is_simple(int rank, const int32_t* cfg) { return is_simple(NDC(cfg, rank)) ? 1 : 0; }
int64_t orc_index_of_index(int rank, const int32_t* cfg, int64_t i) {
    NDC c(cfg, rank);
    int idx[MAX_RANK];
    c.indices_of_index(i, idx);
    return c.index_of_indices(idx);
}

void orc_gaussian_from(int64_t seed, double* out2) { gaussian_from(uint64_t(seed), out2); }

// CPURandomization.fillRandomly for float[]/double[] (CPURandomization.java:112-136, :137-152):
// element pair (i, i+1) = gaussianFrom(seed + i).
void orc_fill_randomly(int dtype, void* out, int64_t n, int64_t seed) {
    double g[2];
    for (int64_t i = 0; i < n; i += 2) {
        gaussian_from(uint64_t(seed + i), g);
        if (dtype == 0) {
            ((float*)out)[i] = float(g[0]);
            if (i + 1 < n) ((float*)out)[i + 1] = float(g[1]);
        } else {
            ((double*)out)[i] = g[0];
            if (i + 1 < n) ((double*)out)[i + 1] = g[1];
        }
    }
}

}  // extern "C"

// ---- MatMul and DotProduct (the CPU implementations the `@` and `dot` operations run) -------------------------------------
// CPUMatMul (implementations/matmul/CPUMatMul.java:30-110) hands dense row-major F32/F64 matrices to
// GEMM.operationForF32/F64 (operations/linear/internal/blas/GEMM.java:55-125); every variant it picks adds the products of one
// output in rising order of the common index into a product array that starts at zero -- the general row-major one
// (partial_F32_MxN_RM, GEMM.java:282-305) as one AXPY per (common index c, left row j):
// product[j, :] += left[j, c] * right[c, :] (AXPY.java: y[i] += a * x[i], a separate multiply and add). Restated as such.
template <class T>
static void matmul_rm(T* product, const T* left, const T* right, int64_t rows, int64_t complexity, int64_t cols) {
    for (int64_t i = 0; i < rows * cols; i++) product[i] = T(0);
    for (int64_t c = 0; c < complexity; c++)
        for (int64_t j = 0; j < rows; j++) {
            const T a = left[c + j * complexity];
            T* y = product + j * cols;
            const T* x = right + c * cols;
            for (int64_t i = 0; i < cols; i++) y[i] = y[i] + a * x[i];
        }
}
extern "C" void orc_matmul(int dtype, void* product, const void* left, const void* right, int64_t rows, int64_t complexity, int64_t cols) {
    if (dtype == 0) matmul_rm((float*)product, (const float*)left, (const float*)right, rows, complexity, cols);
    else matmul_rm((double*)product, (const double*)left, (const double*)right, rows, complexity, cols);
}

// CPUDot (implementations/linear/CPUDot.java:11-90) -> DOT.unrolled04 (operations/linear/internal/blas/DOT.java:148-179): four
// partial sums over the elements i % 4 == 0..3 of the largest multiple of four, the remainder into the first one, then
// sum0 + sum1 + sum2 + sum3 left to right.
template <class T>
static T dot_unrolled04(const T* a, const T* b, int64_t n) {
    const int64_t remainder = n % 4;
    T s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    int64_t i = 0;
    for (const int64_t lim = n - remainder; i < lim; i += 4) {
        s0 += a[i] * b[i];
        s1 += a[i + 1] * b[i + 1];
        s2 += a[i + 2] * b[i + 2];
        s3 += a[i + 3] * b[i + 3];
    }
    for (; i < n; i++) s0 += a[i] * b[i];
    return s0 + s1 + s2 + s3;
}
extern "C" double orc_dot(int dtype, const void* a, const void* b, int64_t n) {
    if (dtype == 0) return double(dot_unrolled04((const float*)a, (const float*)b, n));
    return dot_unrolled04((const double*)a, (const double*)b, n);
}
