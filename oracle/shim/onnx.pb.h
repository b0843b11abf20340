// Stand-in for the protobuf-generated <onnx.pb.h>, used ONLY to compile the reference's
// src/sparse_onnx.cpp unchanged into oracle/_ref/ (libprotobuf and protoc are not available).
// It is a minimal protobuf wire-format reader that offers the accessor subset that file uses.
// Field numbers are those of the public ONNX schema (onnx.proto).  Test infrastructure only.
#pragma once
#include <string>
#include <vector>
#include <cstdint>
#include <cstring>
#include <istream>
#include <iterator>
namespace onnx {
struct Rd { const uint8_t* p; const uint8_t* e;
  bool ok() const { return p < e; }
  uint64_t varint(){ uint64_t v=0; int s=0; while(p<e){ uint8_t b=*p++; v|=uint64_t(b&0x7f)<<s; if(!(b&0x80))break; s+=7;} return v; }
  Rd sub(){ uint64_t n=varint(); Rd r{p,p+n}; p+=n; return r; }
  void skip(int wt){ if(wt==0)varint(); else if(wt==1)p+=8; else if(wt==2){uint64_t n=varint(); p+=n;} else if(wt==5)p+=4; }
  std::string str(){ Rd r=sub(); return std::string((const char*)r.p,(const char*)r.e);} };
template<class T> struct Rep { std::vector<T> v; auto begin() const {return v.begin();} auto end() const {return v.end();} };
struct Dimension { bool has=false; int64_t val=0; bool has_dim_value() const {return has;} int64_t dim_value() const {return val;}
  void parse(Rd r){ while(r.ok()){ uint64_t k=r.varint(); int f=k>>3,wt=k&7; if(f==1&&wt==0){has=true; val=(int64_t)r.varint();} else r.skip(wt);} } };
struct TensorShapeProto { std::vector<Dimension> d; int dim_size() const {return (int)d.size();} const Dimension& dim(int i) const {return d[i];}
  void parse(Rd r){ while(r.ok()){ uint64_t k=r.varint(); int f=k>>3,wt=k&7; if(f==1&&wt==2){Dimension x; x.parse(r.sub()); d.push_back(x);} else r.skip(wt);} } };
struct TypeTensor { TensorShapeProto s; const TensorShapeProto& shape() const {return s;}
  void parse(Rd r){ while(r.ok()){ uint64_t k=r.varint(); int f=k>>3,wt=k&7; if(f==2&&wt==2) s.parse(r.sub()); else r.skip(wt);} } };
struct TypeProto { TypeTensor t; const TypeTensor& tensor_type() const {return t;}
  void parse(Rd r){ while(r.ok()){ uint64_t k=r.varint(); int f=k>>3,wt=k&7; if(f==1&&wt==2) t.parse(r.sub()); else r.skip(wt);} } };
struct ValueInfoProto { std::string n; TypeProto ty; const std::string& name() const {return n;} const TypeProto& type() const {return ty;}
  void parse(Rd r){ while(r.ok()){ uint64_t k=r.varint(); int f=k>>3,wt=k&7; if(f==1&&wt==2) n=r.str(); else if(f==2&&wt==2) ty.parse(r.sub()); else r.skip(wt);} } };
struct TensorProto { std::vector<int64_t> dm; std::string n, raw; std::vector<float> fd; bool hasraw=false;
  const std::string& name() const {return n;} int dims_size() const {return (int)dm.size();} int64_t dims(int i) const {return dm[i];}
  bool has_raw_data() const {return hasraw;} const std::string& raw_data() const {return raw;}
  int float_data_size() const {return (int)fd.size();} float float_data(int i) const {return fd[i];}
  void parse(Rd r){ while(r.ok()){ uint64_t k=r.varint(); int f=k>>3,wt=k&7;
    if(f==1&&wt==0) dm.push_back((int64_t)r.varint()); else if(f==1&&wt==2){Rd s=r.sub(); while(s.ok()) dm.push_back((int64_t)s.varint());}
    else if(f==8&&wt==2) n=r.str(); else if(f==9&&wt==2){raw=r.str(); hasraw=true;}
    else if(f==4&&wt==2){Rd s=r.sub(); while(s.ok()){float x; std::memcpy(&x,s.p,4); s.p+=4; fd.push_back(x);}} else if(f==4&&wt==5){float x; std::memcpy(&x,r.p,4); r.p+=4; fd.push_back(x);}
    else r.skip(wt);} } };
struct AttributeProto { std::string n; int64_t iv=0; std::vector<int64_t> iv_s;
  const std::string& name() const {return n;} int64_t i() const {return iv;} int ints_size() const {return (int)iv_s.size();} int64_t ints(int k) const {return iv_s[k];}
  void parse(Rd r){ while(r.ok()){ uint64_t k=r.varint(); int f=k>>3,wt=k&7; if(f==1&&wt==2) n=r.str(); else if(f==3&&wt==0) iv=(int64_t)r.varint();
    else if(f==8&&wt==0) iv_s.push_back((int64_t)r.varint()); else if(f==8&&wt==2){Rd s=r.sub(); while(s.ok()) iv_s.push_back((int64_t)s.varint());} else r.skip(wt);} } };
struct NodeProto { std::vector<std::string> in,out; std::string op; Rep<AttributeProto> at;
  const std::string& op_type() const {return op;} const std::string& input(int i) const {return in[i];} const std::string& output(int i) const {return out[i];}
  int input_size() const {return (int)in.size();} const Rep<AttributeProto>& attribute() const {return at;}
  void parse(Rd r){ while(r.ok()){ uint64_t k=r.varint(); int f=k>>3,wt=k&7; if(f==1&&wt==2) in.push_back(r.str()); else if(f==2&&wt==2) out.push_back(r.str());
    else if(f==4&&wt==2) op=r.str(); else if(f==5&&wt==2){AttributeProto a; a.parse(r.sub()); at.v.push_back(a);} else r.skip(wt);} } };
struct GraphProto { Rep<NodeProto> nd; Rep<TensorProto> init; Rep<ValueInfoProto> in,out;
  const Rep<TensorProto>& initializer() const {return init;} int initializer_size() const {return (int)init.v.size();}
  const Rep<ValueInfoProto>& input() const {return in;} int output_size() const {return (int)out.v.size();} const ValueInfoProto& output(int i) const {return out.v[i];}
  size_t node_size() const {return nd.v.size();} const NodeProto& node(size_t i) const {return nd.v[i];}
  void parse(Rd r){ while(r.ok()){ uint64_t k=r.varint(); int f=k>>3,wt=k&7; if(f==1&&wt==2){NodeProto n; n.parse(r.sub()); nd.v.push_back(std::move(n));}
    else if(f==5&&wt==2){TensorProto t; t.parse(r.sub()); init.v.push_back(std::move(t));} else if(f==11&&wt==2){ValueInfoProto v; v.parse(r.sub()); in.v.push_back(v);}
    else if(f==12&&wt==2){ValueInfoProto v; v.parse(r.sub()); out.v.push_back(v);} else r.skip(wt);} } };
struct ModelProto { GraphProto g; std::string buf; const GraphProto& graph() const {return g;}
  bool ParseFromIstream(std::istream* is){ buf.assign(std::istreambuf_iterator<char>(*is),{}); Rd r{(const uint8_t*)buf.data(),(const uint8_t*)buf.data()+buf.size()};
    while(r.ok()){ uint64_t k=r.varint(); int f=k>>3,wt=k&7; if(f==7&&wt==2) g.parse(r.sub()); else r.skip(wt);} return true; } };
}
