// Stand-in for glog, enough to compile the reference (golden outputs of the tests, reference arm of the benchmark).
#pragma once
#include <cstdlib>
#include <iostream>
#include <sstream>
#include <string>
namespace golden_glog {
struct Sink { bool fatal; std::ostringstream os; explicit Sink(bool f):fatal(f){} ~Sink(){ if(fatal){ std::cerr<<os.str()<<std::endl; std::abort(); } else if(!os.str().empty()) std::cerr<<os.str()<<std::endl; } template<class T> Sink& operator<<(const T& v){ os<<v; return *this; } };
struct Voidify { void operator&(Sink&){} void operator&(const Sink&){} };
}
#define LOG(sev) ::golden_glog::Sink(std::string(#sev)=="FATAL")
#define CHECK(c) (c) ? (void)0 : ::golden_glog::Voidify() & ::golden_glog::Sink(true) << "CHECK failed: " #c " "
#define CHECK_OP(a,b,op) CHECK((a) op (b))
#define CHECK_EQ(a,b) CHECK_OP(a,b,==)
#define CHECK_NE(a,b) CHECK_OP(a,b,!=)
#define CHECK_GT(a,b) CHECK_OP(a,b,>)
#define CHECK_GE(a,b) CHECK_OP(a,b,>=)
#define CHECK_LT(a,b) CHECK_OP(a,b,<)
#define CHECK_LE(a,b) CHECK_OP(a,b,<=)
namespace google { inline void InitGoogleLogging(const char*){} }
static bool FLAGS_alsologtostderr = true; static std::string FLAGS_log_dir;
