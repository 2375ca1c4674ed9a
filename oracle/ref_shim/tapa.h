// Stand-in for <tapa.h>: streams are unbounded FIFOs (C-simulation semantics), mmap is a pointer.
// Enough for calling the operator templates one after another on pre-filled streams.
#pragma once
#include <deque>
#include <cstdio>
#include <cstdlib>
namespace tapa {
template <class T> struct sbase { std::deque<T> q; };
template <class T> struct istream : virtual sbase<T> {
    T read() {
        if (this->q.empty()) { fprintf(stderr, "tapa shim: read on empty stream\n"); abort(); }
        T t = this->q.front(); this->q.pop_front(); return t;
    }
    bool try_read(T& t) { if (this->q.empty()) return false; t = read(); return true; }
    bool empty() const { return this->q.empty(); }
};
template <class T> struct ostream : virtual sbase<T> {
    void write(const T& t) { this->q.push_back(t); }
    bool try_write(const T& t) { write(t); return true; }
};
template <class T, int D = 2> struct stream : istream<T>, ostream<T> { stream(const char* = "") {} };
template <class T, int N> struct istreams { stream<T>* s[N]; istream<T>& operator[](int i) { return *s[i]; } };
template <class T, int N> struct ostreams { stream<T>* s[N]; ostream<T>& operator[](int i) { return *s[i]; } };
template <class T> struct mmap { T* p; mmap(T* p_) : p(p_) {} T& operator[](long i) { return p[i]; } };
}
