// Stand-in for Vitis HLS <hls_stream.h>: an unbounded FIFO, as in C simulation.
#pragma once
#include <deque>
namespace hls {
template <class T> struct stream {
    std::deque<T> q;
    stream(const char* = "") {}
    T read() { T t = q.front(); q.pop_front(); return t; }
    void write(const T& t) { q.push_back(t); }
    bool empty() const { return q.empty(); }
};
}
