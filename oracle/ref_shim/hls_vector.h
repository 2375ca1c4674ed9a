// Stand-in for Vitis HLS <hls_vector.h>: fixed-size array with scalar broadcast construction.
#pragma once
namespace hls {
template <class T, int N> struct vector {
    T d[N];
    vector() { for (int i = 0; i < N; i++) d[i] = T(); }
    template <class S> vector(const S& s) { for (int i = 0; i < N; i++) d[i] = T(s); }
    T& operator[](int i) { return d[i]; }
    const T& operator[](int i) const { return d[i]; }
};
}
