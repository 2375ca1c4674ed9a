// Stand-in for Vitis HLS <ap_int.h>: W<=63-bit two's-complement / unsigned integers kept
// sign- or zero-extended in a 64-bit word, with range(), (hi,lo), [bit], += and comma
// concatenation usable as rvalue and lvalue. Integer * float converts the integer to
// float first (through long long), which is what the operator code relies on.
#pragma once
// minimal bit-accurate ap_int/ap_uint (W<=63) : range(), (hi,lo), [bit], comma-concat (lvalue + rvalue)
template<int W> struct ap_uint; template<int W> struct ap_int;
template<int W,bool S> struct ap_base {
  long long v=0;
  static long long norm(long long x){ unsigned long long m=(W>=64)?~0ULL:((1ULL<<W)-1); unsigned long long u=(unsigned long long)x&m; if(S && W<64 && (u>>(W-1))) u|=~m; return (long long)u; }
  unsigned long long bits() const { unsigned long long m=(W>=64)?~0ULL:((1ULL<<W)-1); return (unsigned long long)v&m; }
  void setbits(unsigned long long u){ v=norm((long long)u); }
  operator long long() const {return v;}
  struct rng { ap_base& b; int hi,lo;
    unsigned long long get() const { int w=hi-lo+1; unsigned long long m=(w>=64)?~0ULL:((1ULL<<w)-1); return (b.bits()>>lo)&m; }
    template<int W2> operator ap_int<W2>() const; template<int W2> operator ap_uint<W2>() const;
    template<class T> rng& operator=(const T& x){ int w=hi-lo+1; unsigned long long m=((w>=64)?~0ULL:((1ULL<<w)-1)); unsigned long long u=b.bits(); u=(u&~(m<<lo))|((((unsigned long long)(long long)x)&m)<<lo); b.setbits(u); return *this; } };
  rng range(int hi,int lo){ return rng{*this,hi,lo}; } rng operator()(int hi,int lo){ return rng{*this,hi,lo}; }
  bool operator[](int i) const { return (bits()>>i)&1; }
  template<class T> ap_base& operator+=(const T& x){ v=norm(v+(long long)x); return *this; }
};
template<int W> struct ap_int : ap_base<W,true> { using B=ap_base<W,true>;
  ap_int()=default; ap_int(int x){this->v=B::norm(x);} ap_int(long long x){this->v=B::norm(x);} ap_int(unsigned long long x){this->v=B::norm((long long)x);} ap_int(bool x){this->v=B::norm(x);} ap_int(float x){this->v=B::norm((long long)x);} ap_int(double x){this->v=B::norm((long long)x);}
  template<int W2,bool S2> ap_int(const ap_base<W2,S2>& o){this->v=B::norm(o.v);} };
template<int W> struct ap_uint : ap_base<W,false> { using B=ap_base<W,false>;
  ap_uint()=default; ap_uint(int x){this->v=B::norm(x);} ap_uint(long long x){this->v=B::norm(x);} ap_uint(unsigned long long x){this->v=B::norm((long long)x);} ap_uint(bool x){this->v=B::norm(x);} ap_uint(float x){this->v=B::norm((long long)x);} ap_uint(double x){this->v=B::norm((long long)x);}
  template<int W2,bool S2> ap_uint(const ap_base<W2,S2>& o){this->v=B::norm(o.v);} };
template<int W,bool S> template<int W2> ap_base<W,S>::rng::operator ap_int<W2>() const { return ap_int<W2>((long long)get()); }
template<int W,bool S> template<int W2> ap_base<W,S>::rng::operator ap_uint<W2>() const { return ap_uint<W2>((long long)get()); }
// concatenation: (hi_part, lo_part)
template<int W> struct cat_val : ap_base<W,false> { };
template<class H,class L,int WH,int WL> struct cat_ref { H& h; L& l; 
  unsigned long long get() const { return (gethi()<<WL)|getlo(); }
  unsigned long long gethi() const { return h.bits(); } unsigned long long getlo() const { return l.bits(); }
  template<int W2> operator ap_uint<W2>() const { return ap_uint<W2>((long long)get()); }
  template<int W2> operator ap_int<W2>() const { return ap_int<W2>((long long)get()); }
  unsigned long long bits() const { return get(); }
  void setbits(unsigned long long u){ l.setbits(u & ((WL>=64)?~0ULL:((1ULL<<WL)-1))); h.setbits(u>>WL); }
  template<int W2,bool S2> cat_ref& operator=(const ap_base<W2,S2>& x){ setbits(x.bits()); return *this; } };
template<int A,bool SA,int B,bool SB> cat_ref<ap_base<A,SA>,ap_base<B,SB>,A,B> operator,(ap_base<A,SA>& a, ap_base<B,SB>& b){ return {a,b}; }
template<class H,class L,int WH,int WL,int B,bool SB> cat_ref<cat_ref<H,L,WH,WL>,ap_base<B,SB>,WH+WL,B> operator,(cat_ref<H,L,WH,WL> a, ap_base<B,SB>& b){ static thread_local cat_ref<H,L,WH,WL>* keep; keep=new cat_ref<H,L,WH,WL>(a); return {*keep,b}; }
